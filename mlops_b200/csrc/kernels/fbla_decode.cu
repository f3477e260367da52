// Launchers of the decode passes (bodies: fbla_decode.cuh).
#include "fbla_decode.cuh"
#include <stdio.h>

namespace fbla {
template <int CB, int FB, int QG, int DEAL>
__global__ void __launch_bounds__(32 * CoarseShape<CB>::TOTAL, 1) coarse_kernel(const fbla_k_decode a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  coarse_item<CB, FB, QG, DEAL>(a, smem_raw);
}

template <int QG>
__global__ void __launch_bounds__(256) select_kernel(const fbla_k_decode a) {
  select_item<QG>(a, nullptr);
}

template <int CB, int FB, int QG>
__global__ void __launch_bounds__(32 * RefineShape<CB, FB>::WARPS, 1) refine_kernel(const fbla_k_decode a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  refine_item<CB, FB, QG>(a, smem_raw);
}

template <int QG>
__global__ void __launch_bounds__(512, 2) merge_kernel(const fbla_k_decode a) {
  merge_item<QG>(a, nullptr);
}

// a launch that may begin while the previous kernel of the stream still runs (the kernel calls wait_previous_pass)
template <class... P, class... A>
cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

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

constexpr int REFINE_SMEM_MAX = 220 * 1024;  // dynamic shared memory of the refine pass (its ring + the slice prefix)
template <int CB, int FB, int QG> cudaError_t launch_all(const fbla_k_decode &a, cudaStream_t stream) {
  const int vheads = a.batch * a.kv_heads * a.vg;
  const size_t csm = sizeof(CoarseSmem<CB>);
  const size_t rsm = sizeof(RefineWarp<CB, FB>) * RefineShape<CB, FB>::WARPS + sizeof(int) * ((size_t)vheads * a.nslices + 1);
  static thread_local int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_LENGTHS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csm);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_FIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csm);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_COST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csm);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(refine_kernel<CB, FB, QG>, cudaFuncAttributeMaxDynamicSharedMemorySize, REFINE_SMEM_MAX);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = 1;
  }
  if (rsm > REFINE_SMEM_MAX) return cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  if (a.status_cleared && a.phase != 2) {  // ordered before every report of this call (a bounded wait that gives up); a shard's second
                                           // phase keeps what its first phase may have reported
    e = cudaMemsetAsync(a.status, 0, 16, stream);
    if (e != cudaSuccess) return e;
  }
  if (a.phase != 2) {
    if (a.deal == FBLA_K_DEAL_LENGTHS) coarse_kernel<CB, FB, QG, FBLA_K_DEAL_LENGTHS><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
    else if (a.deal == FBLA_K_DEAL_FIXED) coarse_kernel<CB, FB, QG, FBLA_K_DEAL_FIXED><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
    else coarse_kernel<CB, FB, QG, FBLA_K_DEAL_COST><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = launch_dependent(select_kernel<QG>, dim3(a.phase == 1 ? 1 : a.nslices, vheads), dim3(256), 0, stream, a);
    if (a.phase == 1) return e;
  } else {
    select_kernel<QG><<<dim3(a.nslices, vheads), 256, 0, stream>>>(a);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = launch_dependent(refine_kernel<CB, FB, QG>, dim3(a.refine_ctas), dim3(32 * RefineShape<CB, FB>::WARPS), rsm, stream, a);
  if (e == cudaSuccess) e = launch_dependent(merge_kernel<QG>, dim3(vheads * QG), dim3(512), 0, stream, a);
  return e;
}

// one pass alone, as an ordinary launch (no overlap with its neighbours): for measurements pass by pass
template <int CB, int FB, int QG> cudaError_t launch_one(const fbla_k_decode &a, int pass, cudaStream_t stream) {
  const int vheads = a.batch * a.kv_heads * a.vg;
  const size_t csm = sizeof(CoarseSmem<CB>);
  const size_t rsm = sizeof(RefineWarp<CB, FB>) * RefineShape<CB, FB>::WARPS + sizeof(int) * ((size_t)vheads * a.nslices + 1);
  if (rsm > REFINE_SMEM_MAX) return cudaErrorInvalidValue;
  switch (pass) {
    case 0:
      if (a.deal == FBLA_K_DEAL_LENGTHS) coarse_kernel<CB, FB, QG, FBLA_K_DEAL_LENGTHS><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
      else if (a.deal == FBLA_K_DEAL_FIXED) coarse_kernel<CB, FB, QG, FBLA_K_DEAL_FIXED><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
      else coarse_kernel<CB, FB, QG, FBLA_K_DEAL_COST><<<a.coarse_ctas, 32 * CoarseShape<CB>::TOTAL, csm, stream>>>(a);
      break;
    case 1: select_kernel<QG><<<dim3(a.nslices, vheads), 256, 0, stream>>>(a); break;
    case 2: refine_kernel<CB, FB, QG><<<a.refine_ctas, 32 * RefineShape<CB, FB>::WARPS, rsm, stream>>>(a); break;
    case 3: merge_kernel<QG><<<vheads * QG, 512, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <int CB, int FB, int QG> cudaError_t passes_of(const fbla_k_decode &a, fbla_k_pass *p) {
  const int vheads = a.batch * a.kv_heads * a.vg;
  const size_t csm = sizeof(CoarseSmem<CB>) + 128;
  const size_t rsm = sizeof(RefineWarp<CB, FB>) * RefineShape<CB, FB>::WARPS + sizeof(int) * ((size_t)vheads * a.nslices + 1) + 128;
  if (rsm - 128 > REFINE_SMEM_MAX) return cudaErrorInvalidValue;
  char e[96];
  snprintf(e, sizeof e, "fbla::coarse_item<%d, %d, %d, %d>", CB, FB, QG, (int)a.deal);
  cudaError_t st = a.deal == FBLA_K_DEAL_LENGTHS ? pass_of(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_LENGTHS>, a.coarse_ctas, 1, 32 * CoarseShape<CB>::TOTAL, csm, e, p + 0)
                   : a.deal == FBLA_K_DEAL_FIXED ? pass_of(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_FIXED>, a.coarse_ctas, 1, 32 * CoarseShape<CB>::TOTAL, csm, e, p + 0)
                                                 : pass_of(coarse_kernel<CB, FB, QG, FBLA_K_DEAL_COST>, a.coarse_ctas, 1, 32 * CoarseShape<CB>::TOTAL, csm, e, p + 0);
  snprintf(e, sizeof e, "fbla::select_item<%d>", QG);
  if (st == cudaSuccess) st = pass_of(select_kernel<QG>, a.nslices, vheads, 256, 0, e, p + 1);
  snprintf(e, sizeof e, "fbla::refine_item<%d, %d, %d>", CB, FB, QG);
  if (st == cudaSuccess) st = pass_of(refine_kernel<CB, FB, QG>, a.refine_ctas, 1, 32 * RefineShape<CB, FB>::WARPS, rsm, e, p + 2);
  snprintf(e, sizeof e, "fbla::merge_item<%d>", QG);
  if (st == cudaSuccess) st = pass_of(merge_kernel<QG>, vheads * QG, 1, 512, 0, e, p + 3);
  return st;
}

// a row's shares summed over the shards -> the BF16 output
__global__ void __launch_bounds__(128) combine_kernel(const float *partial, uint16_t *out) {
  const float *p = partial + (size_t)blockIdx.x * PSTRIDE;
  out[(size_t)blockIdx.x * D + threadIdx.x] = f32_to_bf16(__fdividef(p[threadIdx.x], p[D]));
}

// R_total[i] = log2 sum_s 2^(mass[s][i]) over the shards (masses of -inf contribute nothing)
__global__ void __launch_bounds__(128) total_mass_kernel(const float *mass, float *total, int shards, int rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  float mx = -INFINITY;
  for (int s = 0; s < shards; ++s) mx = fmaxf(mx, mass[(size_t)s * rows + i]);
  float sum = 0.f;
  for (int s = 0; s < shards; ++s) { const float m = mass[(size_t)s * rows + i]; if (m != -INFINITY) sum += ex2(m - mx); }
  total[i] = mx + lg2(sum);
}

}  // namespace fbla

extern "C" cudaError_t fbla_k_total_mass_launch(const float *mass, float *total, int shards, int rows, cudaStream_t stream) {
  fbla::total_mass_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(mass, total, shards, rows);
  return cudaGetLastError();
}

extern "C" cudaError_t fbla_k_combine_launch(const float *partial, uint16_t *out, int rows, cudaStream_t stream) {
  fbla::combine_kernel<<<rows, 128, 0, stream>>>(partial, out);
  return cudaGetLastError();
}

extern "C" long long fbla_k_refine_entry_limit(int cb) {
  using namespace fbla;
  const size_t ring = cb == 3 ? sizeof(RefineWarp<3, 3>) * RefineShape<3, 3>::WARPS : sizeof(RefineWarp<4, 2>) * RefineShape<4, 2>::WARPS;
  return (long long)((REFINE_SMEM_MAX - ring) / sizeof(int)) - 1;
}

extern "C" cudaError_t fbla_k_decode_shape(fbla_k_decode *a) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  a->coarse_ctas = sms;
  a->coarse_warps = fbla::CoarseShape<4>::TOTAL;  // (the larger of the two layouts: what the scratch is sized for)
  a->refine_ctas = sms;
  a->refine_warps = fbla::RefineShape<4, 2>::WARPS;
  return cudaSuccess;
}

// How the coarse CTAs' warps share the work (see split_of, deal_of), from the tokens a row has at most:
//   by the lengths when the BF16 windows would get three or more of a CTA's eight warps (contexts up to about 4 700 tokens);
//   else seven streaming warps and one window warp per CTA, or every warp an equal cost share of windows and groups --
//   whichever leaves a streaming warp fewer groups, counted as the kernels deal them (whole groups per warp), with 5 %
//   against the deal by cost: its eight streaming warps per CTA run a group that much slower than seven beside a window
//   warp do. Measured on B200, by cost against seven + one: batch 1 x 128K tokens 80.0 -> 75.3 us per step in 3+3 and
//   65.7 -> 61.6 in 4+2 (7 groups per warp instead of 8), batch 64 x 1K..64K 2.07 -> 2.02 ms, but batch 8 x 16K 120.0 ->
//   123.9 (8 groups per warp either way).
extern "C" void fbla_k_decode_split(fbla_k_decode *a, long long tokens) {
  const int total = (a->cb == 4 ? fbla::CoarseShape<4>::TOTAL : fbla::CoarseShape<3>::TOTAL);
  const long long groups = (tokens + fbla::G - 1) / fbla::G, S = groups > 2 ? groups - 2 : 0;
  const long long W = groups <= 1 ? (tokens + fbla::S - 1) / fbla::S : 2 * fbla::SBG;  // (a full open window: the choice is monotone in tokens)
  const bool by_lengths = S == 0 || (2 * total * W + S + W) / (2 * (S + W)) >= 3;
  const long long heads = (long long)a->batch * a->kv_heads * a->vg, ctas = a->coarse_ctas > 0 ? a->coarse_ctas : 148;
  // groups a streaming warp takes: seven + one; by cost (deal_of's share, a whole number of groups)
  const long long fixed = (heads * S + ctas * (total - 1) - 1) / (ctas * (total - 1));
  const long long cost = (fbla::GROUP_COST * heads * S + fbla::WINDOW_COST * heads * W + fbla::GROUP_COST * ctas * total - 1) / (fbla::GROUP_COST * ctas * total);
  a->coarse_warps = total;
  a->deal = by_lengths ? FBLA_K_DEAL_LENGTHS : 21 * cost < 20 * fixed ? FBLA_K_DEAL_COST : FBLA_K_DEAL_FIXED;
  // Folding the warps' partial rows per CTA costs the coarse pass a barrier and a few microseconds at its very end and saves
  // the later passes their walk over the rows: it pays when a virtual head is spread over many warps, i.e. when there are
  // few heads (measured on B200: batch 1 x 8 KV heads at 128K tokens -4.5 us per step, batch 8 x 8 heads at 16K +3 us).
  a->fold = !by_lengths && a->batch * a->kv_heads * a->vg <= 32;
}

extern "C" void fbla_k_decode_split_of(int cb, int batch, int kv_heads, int vg, long long tokens, int *deal, int *fold) {
  fbla_k_decode a = {};
  a.cb = cb; a.batch = batch; a.kv_heads = kv_heads; a.vg = vg;
  a.coarse_ctas = 148;  // (the shape of a B200; a caller with a device takes it from fbla_k_decode_shape)
  fbla_k_decode_split(&a, tokens);
  *deal = a.deal;
  *fold = a.fold;
}

extern "C" cudaError_t fbla_k_decode_launch(const fbla_k_decode *a, cudaStream_t stream) {
  using namespace fbla;
  if (a->cb == 3) {
    switch (a->qg) {
      case 1: return launch_all<3, 3, 1>(*a, stream);
      case 2: return launch_all<3, 3, 2>(*a, stream);
      default: return launch_all<3, 3, 4>(*a, stream);
    }
  }
  switch (a->qg) {
    case 1: return launch_all<4, 2, 1>(*a, stream);
    case 2: return launch_all<4, 2, 2>(*a, stream);
    default: return launch_all<4, 2, 4>(*a, stream);
  }
}

// (after one whole fbla_k_decode_launch on this device: that call sets the kernels' shared-memory attributes)
extern "C" cudaError_t fbla_k_decode_pass_launch(const fbla_k_decode *a, int pass, cudaStream_t stream) {
  using namespace fbla;
  if (a->cb == 3) {
    switch (a->qg) {
      case 1: return launch_one<3, 3, 1>(*a, pass, stream);
      case 2: return launch_one<3, 3, 2>(*a, pass, stream);
      default: return launch_one<3, 3, 4>(*a, pass, stream);
    }
  }
  switch (a->qg) {
    case 1: return launch_one<4, 2, 1>(*a, pass, stream);
    case 2: return launch_one<4, 2, 2>(*a, pass, stream);
    default: return launch_one<4, 2, 4>(*a, pass, stream);
  }
}

extern "C" cudaError_t fbla_k_decode_passes(const fbla_k_decode *a, fbla_k_pass info[4]) {
  using namespace fbla;
  if (a->cb == 3) {
    switch (a->qg) {
      case 1: return passes_of<3, 3, 1>(*a, info);
      case 2: return passes_of<3, 3, 2>(*a, info);
      default: return passes_of<3, 3, 4>(*a, info);
    }
  }
  switch (a->qg) {
    case 1: return passes_of<4, 2, 1>(*a, info);
    case 2: return passes_of<4, 2, 2>(*a, info);
    default: return passes_of<4, 2, 4>(*a, info);
  }
}
