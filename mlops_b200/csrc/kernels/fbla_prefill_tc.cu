// Launchers of the tensor-core prefill attention (body: fbla_prefill_tc.cuh).
#include "fbla_prefill_tc.cuh"
#include <stdlib.h>
#include <string.h>
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
namespace tc {
template <int CB, int FB>
__global__ void __launch_bounds__(THREADS, 1) attend_tc_kernel(const fbla_k_prefill a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  attend_tc_item<CB, FB>(a, smem_raw);
}
}  // namespace tc
}  // namespace fbla

extern "C" int fbla_k_attend_tc_status(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, fbla::tc::g_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(fbla::tc::g_status, &zero, sizeof(int));
  return v;
}

extern "C" cudaError_t fbla_k_attend_tc_launch(const fbla_k_prefill *a, cudaStream_t stream) {
  using namespace fbla::tc;
  const int qg = a->q_heads / a->kv_heads;
  const dim3 grid((a->count * qg + CTA_ROWS - 1) / CTA_ROWS, a->batch * a->kv_heads);
  const size_t smem = sizeof(Smem) + 1024;
  static thread_local int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attend_tc_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attend_tc_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = 1;
  }
  if (a->cb == 3) attend_tc_kernel<3, 3><<<grid, THREADS, smem, stream>>>(*a);
  else attend_tc_kernel<4, 2><<<grid, THREADS, smem, stream>>>(*a);
  return cudaGetLastError();
}

extern "C" int fbla_k_attend_plan(const fbla_k_prefill *a, fbla_k_prefill args[2], int tensor[2]) {
  static const bool rows_only = [] { const char *e = getenv("MLOPS_FBLA_PREFILL"); return e && !strcmp(e, "rows"); }();
  const int rows = a->count * (a->q_heads / a->kv_heads);  // (with a device count: the ceiling)
  args[0] = *a;
  args[0].tc_min_rows = 0;
  if (rows_only || rows < FBLA_K_TC_MIN_ROWS) { tensor[0] = 0; return 1; }
  tensor[0] = 1;
  if (!a->dcount) return 1;
  args[0].tc_min_rows = FBLA_K_TC_MIN_ROWS;
  args[1] = args[0];
  tensor[1] = 0;
  return 2;
}

extern "C" cudaError_t fbla_k_attend_launch(const fbla_k_prefill *a, cudaStream_t stream) {
  fbla_k_prefill args[2];
  int tensor[2];
  const int n = fbla_k_attend_plan(a, args, tensor);
  cudaError_t e = cudaSuccess;
  for (int i = 0; i < n && e == cudaSuccess; ++i) e = tensor[i] ? fbla_k_attend_tc_launch(&args[i], stream) : fbla_k_attend_rows_launch(&args[i], stream);
  return e;
}

extern "C" cudaError_t fbla_k_attend_tc_pass(const fbla_k_prefill *a, fbla_k_pass *info) {
  using namespace fbla::tc;
  const int qg = a->q_heads / a->kv_heads, rows = a->count * qg, heads = a->batch * a->kv_heads;
  const size_t smem = sizeof(Smem) + 1024;
  if (a->cb == 3) return pass_of(attend_tc_kernel<3, 3>, (rows + CTA_ROWS - 1) / CTA_ROWS, heads, THREADS, smem, "fbla::tc::attend_tc_item<3, 3>", info);
  return pass_of(attend_tc_kernel<4, 2>, (rows + CTA_ROWS - 1) / CTA_ROWS, heads, THREADS, smem, "fbla::tc::attend_tc_item<4, 2>", info);
}
