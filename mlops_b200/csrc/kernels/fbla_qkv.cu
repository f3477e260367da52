// Launchers of the fused QKV step (bodies: fbla_qkv.cuh).
#include "fbla_qkv.cuh"
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
template <bool NORM>
__global__ void __launch_bounds__(256) qkv_token_kernel(const fbla_k_token a) {
  qkv_token_item<NORM>(a, nullptr);
}

template <bool NORM>
__global__ void __launch_bounds__(256) qkv_chunk_kernel(const fbla_k_token a) {
  qkv_chunk_item<NORM>(a, nullptr);
}
}  // namespace fbla

extern "C" cudaError_t fbla_k_qkv_token_launch(const fbla_k_token *a, cudaStream_t stream) {
  const int heads = a->batch * a->kv_heads;
  if (a->q_norm) fbla::qkv_token_kernel<true><<<heads, 256, 0, stream>>>(*a);
  else fbla::qkv_token_kernel<false><<<heads, 256, 0, stream>>>(*a);
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_qkv_chunk_launch(const fbla_k_token *a, cudaStream_t stream) {
  const dim3 grid((a->max_count + fbla::TOK - 1) / fbla::TOK, a->kv_heads);
  if (a->q_norm) fbla::qkv_chunk_kernel<true><<<grid, 256, 0, stream>>>(*a);
  else fbla::qkv_chunk_kernel<false><<<grid, 256, 0, stream>>>(*a);
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_qkv_token_pass(const fbla_k_token *a, fbla_k_pass *info) {
  const int heads = a->batch * a->kv_heads;
  if (a->q_norm) return pass_of(fbla::qkv_token_kernel<true>, heads, 1, 256, 0, "fbla::qkv_token_item<true>", info);
  return pass_of(fbla::qkv_token_kernel<false>, heads, 1, 256, 0, "fbla::qkv_token_item<false>", info);
}

extern "C" cudaError_t fbla_k_qkv_chunk_pass(const fbla_k_token *a, fbla_k_pass *info) {
  const int tiles = (a->max_count + fbla::TOK - 1) / fbla::TOK;
  if (a->q_norm) return pass_of(fbla::qkv_chunk_kernel<true>, tiles, a->kv_heads, 256, 0, "fbla::qkv_chunk_item<true>", info);
  return pass_of(fbla::qkv_chunk_kernel<false>, tiles, a->kv_heads, 256, 0, "fbla::qkv_chunk_item<false>", info);
}
