// Launchers of the close / finish passes (bodies: fbla_close.cuh).
#include "fbla_close.cuh"
#include <stdio.h>

namespace {
template <class K> cudaError_t pass_of(K kernel, int gx, int gy, int threads, size_t smem, const char *entry, fbla_k_pass *p) {
  cudaFuncAttributes fa;
  const cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
  if (e != cudaSuccess) return e;
  p->gx = gx; p->gy = gy; p->gz = 1; p->threads = threads; p->smem_bytes = (int)smem; p->regs = fa.numRegs;
  snprintf(p->entry, sizeof p->entry, "%s", entry);
  return cudaSuccess;
}
}  // namespace

namespace fbla {
template <int CB, int FB>
__global__ void __launch_bounds__(256) close_kernel(const fbla_k_prefill a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  close_item<CB, FB>(a, smem_raw);
}

__global__ void __launch_bounds__(256) finish_kernel(const fbla_k_prefill a) {
  finish_item(a, nullptr);
}
}  // namespace fbla

extern "C" cudaError_t fbla_k_close_launch(const fbla_k_prefill *a, int close_blocks, cudaStream_t stream) {
  if (close_blocks <= 0) return cudaSuccess;
  const dim3 grid(close_blocks, a->batch * a->kv_heads);
  const size_t smem = sizeof(fbla::CloseSmem);
  cudaError_t e;
  if (a->cb == 3) {
    e = cudaFuncSetAttribute(fbla::close_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fbla::close_kernel<3, 3><<<grid, 256, smem, stream>>>(*a);
  } else {
    e = cudaFuncSetAttribute(fbla::close_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fbla::close_kernel<4, 2><<<grid, 256, smem, stream>>>(*a);
  }
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_finish_launch(const fbla_k_prefill *a, cudaStream_t stream) {
  fbla::finish_kernel<<<a->batch * a->kv_heads, 256, 0, stream>>>(*a);
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_close_pass(const fbla_k_prefill *a, int close_blocks, fbla_k_pass *info) {
  const int heads = a->batch * a->kv_heads;
  if (a->cb == 3) return pass_of(fbla::close_kernel<3, 3>, close_blocks, heads, 256, sizeof(fbla::CloseSmem), "fbla::close_item<3, 3>", info);
  return pass_of(fbla::close_kernel<4, 2>, close_blocks, heads, 256, sizeof(fbla::CloseSmem), "fbla::close_item<4, 2>", info);
}

extern "C" cudaError_t fbla_k_finish_pass(const fbla_k_prefill *a, fbla_k_pass *info) {
  return pass_of(fbla::finish_kernel, a->batch * a->kv_heads, 1, 256, 0, "fbla::finish_item", info);
}
