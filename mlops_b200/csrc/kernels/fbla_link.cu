// Sequence-sharded decode without host-side collectives: the two small exchanges of a step (the rows' local masses, then
// the rows' unnormalised sums) as stores into the peers' memory over NVLink.
//
// Every rank owns one "mailbox" buffer that all ranks of the box can address (peer-mapped symmetric memory). A sender
// writes its few KB into its own slot of every mailbox with plain stores, then publishes them with one system-scope
// release store of the step number into that mailbox's flag; a receiver polls its own flags with acquire loads until
// they carry the step number -- a BOUNDED poll: after `spin_limit` tries it records a status and goes on, so a missing
// peer costs a fraction of a second and a marked result, never a hang. Flags are stamped with a step counter that only
// grows, so nothing is ever reset; one buffer per exchange suffices because a rank can only run ahead of a peer by
// less than one step (it needs that peer's data of the current step to finish it).
// No multicast, no multimem, no library collective: peer pointers are only stored to, and read by, these kernels.
// The reference has no multi-GPU path (attention/fbla/src is single-device); this is new.
#include "fbla_device.cuh"
#include "fbla_kernels.h"

namespace fbla {
namespace {

__device__ __forceinline__ void st_release_sys(int *p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int *p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
template <class T> __device__ __forceinline__ T *at(void *base, size_t offset) { return reinterpret_cast<T *>(static_cast<char *>(base) + offset); }

// waits until flag[s] of every rank s carries `epoch` (thread s polls flag s); false where a wait gave up
__device__ __forceinline__ bool await_flags(const fbla_k_link &L, const int *flags, int epoch, int *status, int code) {
  bool ok = true;
  if ((int)threadIdx.x < L.world) {
    unsigned tries = 0;
    while (ld_acquire_sys(flags + threadIdx.x) != epoch) {
      if (++tries > L.spin_limit) { ok = false; atomicCAS(status, 0, code + 16 * (int)threadIdx.x); break; }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok);
}

// the rows' local masses into slot `rank` of every mailbox; opens the step (the step counter moves here)
__global__ void __launch_bounds__(256) push_mass_kernel(const fbla_k_link L) {
  const fbla_k_mailbox M = fbla_k_mailbox_of(L.world, L.rows);
  void *own = L.peer[L.rank];
  const int epoch = *at<int>(own, M.epoch) + 1;
  const float *mass = at<float>(own, M.local_mass);
  for (int p = 0; p < L.world; ++p) {
    float *dst = at<float>(L.peer[p], M.mass_in) + (size_t)L.rank * L.rows;
    for (int i = threadIdx.x; i < L.rows; i += blockDim.x) dst[i] = mass[i];
  }
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    __threadfence_system();
    st_release_sys(at<int>(L.peer[threadIdx.x], M.mass_flag) + L.rank, epoch);
  }
  if (threadIdx.x == 0) *at<int>(own, M.epoch) = epoch;
}

// total[i] = log2 sum over the ranks of 2^mass[s][i], ranks in order (the arithmetic of fbla_k_total_mass_launch)
__global__ void __launch_bounds__(256) gather_mass_kernel(const fbla_k_link L) {
  const fbla_k_mailbox M = fbla_k_mailbox_of(L.world, L.rows);
  void *own = L.peer[L.rank];
  const int epoch = *at<int>(own, M.epoch);
  const bool ok = await_flags(L, at<int>(own, M.mass_flag), epoch, at<int>(own, M.status), 1);
  const float *in = at<float>(own, M.mass_in);
  float *total = at<float>(own, M.total);
  for (int i = threadIdx.x; i < L.rows; i += blockDim.x) {
    float mx = -FBLA_INF;
    for (int s = 0; s < L.world; ++s) mx = fmaxf(mx, __ldcg(in + (size_t)s * L.rows + i));
    float sum = 0.f;
    for (int s = 0; s < L.world; ++s) {
      const float m = __ldcg(in + (size_t)s * L.rows + i);
      if (m != -FBLA_INF) sum += ex2(m - mx);
    }
    total[i] = ok ? mx + lg2(sum) : __int_as_float(0x7fc00000);
  }
}

// the rows' unnormalised sums (o[128], l) into slot `rank` of every mailbox
__global__ void __launch_bounds__(1024) push_partial_kernel(const fbla_k_link L) {
  const fbla_k_mailbox M = fbla_k_mailbox_of(L.world, L.rows);
  void *own = L.peer[L.rank];
  const int epoch = *at<int>(own, M.epoch);
  const int n4 = L.rows * FBLA_K_PSTRIDE / 4;
  const float4 *src = at<float4>(own, M.local_part);
  for (int p = 0; p < L.world; ++p) {
    float4 *dst = at<float4>(L.peer[p], M.part_in) + (size_t)L.rank * n4;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = src[i];
  }
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    __threadfence_system();
    st_release_sys(at<int>(L.peer[threadIdx.x], M.part_flag) + L.rank, epoch);
  }
}

// out[row] = bf16(sum_s o_s / sum_s l_s), ranks in order: every rank computes the same bits
__global__ void __launch_bounds__(128) combine_kernel(const fbla_k_link L, uint16_t *out) {
  const fbla_k_mailbox M = fbla_k_mailbox_of(L.world, L.rows);
  void *own = L.peer[L.rank];
  const int epoch = *at<int>(own, M.epoch), row = blockIdx.x, ch = threadIdx.x;
  const bool ok = await_flags(L, at<int>(own, M.part_flag), epoch, at<int>(own, M.status), 2);
  const float *in = at<float>(own, M.part_in);
  float o = 0.f, l = 0.f;
  for (int s = 0; s < L.world; ++s) {
    const float *p = in + ((size_t)s * L.rows + row) * FBLA_K_PSTRIDE;
    o += __ldcg(p + ch);
    l += __ldcg(p + D);
  }
  out[(size_t)row * D + ch] = ok ? f32_to_bf16(__fdividef(o, l)) : (uint16_t)0x7fc0;
}

}  // namespace
}  // namespace fbla

extern "C" cudaError_t fbla_k_link_push_mass(const fbla_k_link *L, cudaStream_t stream) {
  fbla::push_mass_kernel<<<1, 256, 0, stream>>>(*L);
  return cudaGetLastError();
}
extern "C" cudaError_t fbla_k_link_gather_mass(const fbla_k_link *L, cudaStream_t stream) {
  fbla::gather_mass_kernel<<<1, 256, 0, stream>>>(*L);
  return cudaGetLastError();
}
extern "C" cudaError_t fbla_k_link_push_partial(const fbla_k_link *L, cudaStream_t stream) {
  fbla::push_partial_kernel<<<1, 1024, 0, stream>>>(*L);
  return cudaGetLastError();
}
extern "C" cudaError_t fbla_k_link_combine(const fbla_k_link *L, uint16_t *out, cudaStream_t stream) {
  fbla::combine_kernel<<<L->rows, 128, 0, stream>>>(*L, out);
  return cudaGetLastError();
}
