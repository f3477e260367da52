/* Device entries of the work items (mlops_fbla_items.h), for nvcc or NVRTC (--std=c++17, compute_100a; add the CUDA
 * include directory for cuda_fp16.h). Before including this file the executor defines, in namespace mlops_fbla,
 *   struct Pos  { static __device__ int x(), y(), z(), nx(), ny(), nz(), tid(); static __device__ int ro(const int *); };
 *   __device__ void position(int item, int nx, int ny, int nz);
 * Every thread of the item's CTA calls the entry named by the pass, as entry(args, shared memory).
 * replaces: attention/include/mlops_fbla_items.cuh:1-10 */
#ifndef MLOPS_FBLA_ITEMS_CUH
#define MLOPS_FBLA_ITEMS_CUH
#define FBLA_POS ::mlops_fbla::Pos
#include "../mlops_b200/csrc/kernels/fbla_close.cuh"
#include "../mlops_b200/csrc/kernels/fbla_decode.cuh"
#include "../mlops_b200/csrc/kernels/fbla_prefill_rows.cuh"
#include "../mlops_b200/csrc/kernels/fbla_prefill_tc.cuh"
#include "../mlops_b200/csrc/kernels/fbla_qkv.cuh"
#endif
