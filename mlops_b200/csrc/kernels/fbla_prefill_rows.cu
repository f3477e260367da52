// Launcher of the warp-per-row prefill attention (body: fbla_prefill_rows.cuh).
#include "fbla_prefill_rows.cuh"
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
__global__ void __launch_bounds__(256) attend_rows_kernel(const fbla_k_prefill a) {
  attend_rows_item<CB, FB>(a, nullptr);
}
}  // namespace fbla

extern "C" cudaError_t fbla_k_attend_rows_launch(const fbla_k_prefill *a, cudaStream_t stream) {
  const int qg = a->q_heads / a->kv_heads;
  const dim3 grid((a->count * qg + 7) / 8, a->batch * a->kv_heads);
  if (a->cb == 3) fbla::attend_rows_kernel<3, 3><<<grid, 256, 0, stream>>>(*a);
  else fbla::attend_rows_kernel<4, 2><<<grid, 256, 0, stream>>>(*a);
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_attend_rows_pass(const fbla_k_prefill *a, fbla_k_pass *info) {
  const int rows = a->count * (a->q_heads / a->kv_heads), heads = a->batch * a->kv_heads;
  if (a->cb == 3) return pass_of(fbla::attend_rows_kernel<3, 3>, (rows + 7) / 8, heads, 256, 0, "fbla::attend_rows_item<3, 3>", info);
  return pass_of(fbla::attend_rows_kernel<4, 2>, (rows + 7) / 8, heads, 256, 0, "fbla::attend_rows_item<4, 2>", info);
}
