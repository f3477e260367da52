"""An emulated executor for the work-item interface (include/mlops_fbla_items.h): ctypes mirrors of its structures, the
position policy an executor supplies, run-time compilation of the generated kernels (NVRTC, compute_100a) and, on a GPU,
their launch through the driver API. Modelled on the reference's own emulation (attention/fbla/tests/test_items.cu:115-181)."""
import ctypes
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


class ArgsBlob(ctypes.Union):
    _fields_ = [("align", ctypes.c_longlong), ("bytes", ctypes.c_ubyte * 256)]


class Items(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("items", ctypes.c_int), ("threads", ctypes.c_int), ("smem_bytes", ctypes.c_int), ("regs", ctypes.c_int),
                ("arch", ctypes.c_int), ("entry", ctypes.c_char * 160), ("args_type", ctypes.c_char * 48), ("args_bytes", ctypes.c_int),
                ("args", ArgsBlob), ("geom", ctypes.c_longlong * 32)]


class Range(ctypes.Structure):
    _fields_ = [("arg", ctypes.c_int), ("write", ctypes.c_int), ("offset", ctypes.c_longlong), ("bytes", ctypes.c_longlong),
                ("stride", ctypes.c_longlong), ("rows", ctypes.c_int)]


KINDS = dict(CLOSE=1, TRANSCODE=2, STREAM=3, TC=4, TC_MERGE=5, FINISH=6, COARSE=7, SELECT=8, REFINE=9, MERGE=10, QKV=11, QKV_CHUNK=12)
ARGS = ["Q", "K", "V", "OUT", "COARSE", "FINE", "META", "SINK_K", "SINK_V", "OPEN_K", "OPEN_V", "IMAGES", "SCRATCH", "LENGTH", "COUNT",
        "TQ", "TK", "TV", "TQN", "TKN", "TFREQ", "TQ_OUT", "PART_ML", "PART_O"]

# what an executor defines before including the entries: where the CTA stands, and how device lengths are read
POLICY = r'''
namespace mlops_fbla {
struct PosState { int x, y, z, nx, ny, nz; };
__shared__ PosState pos_state;
struct Pos {
  static __device__ __forceinline__ int x() { return pos_state.x; }
  static __device__ __forceinline__ int y() { return pos_state.y; }
  static __device__ __forceinline__ int z() { return pos_state.z; }
  static __device__ __forceinline__ int nx() { return pos_state.nx; }
  static __device__ __forceinline__ int ny() { return pos_state.ny; }
  static __device__ __forceinline__ int nz() { return pos_state.nz; }
  static __device__ __forceinline__ int tid() { return threadIdx.x; }
  static __device__ __forceinline__ int ro(const int *p) { return __ldcg(p); }
};
__device__ __forceinline__ void position(int item, int nx, int ny, int nz) {
  if (threadIdx.x == 0) { pos_state.x = item % nx; pos_state.y = (item / nx) % ny; pos_state.z = item / (nx * ny);
                          pos_state.nx = nx; pos_state.ny = ny; pos_state.nz = nz; }
}
}
#include "mlops_fbla_items.cuh"
'''


def kernel_source(name, threads, statements, items=None):
    """One executor kernel. items None: CTA i runs item i of the pass. items = the pass's item count: a persistent loop,
    each CTA of a smaller grid walks items blockIdx.x, blockIdx.x + gridDim.x, ... back to back (as the reference's
    emulation runs fewer CTAs than items, attention/fbla/tests/test_items.cu:115-181), so whatever an item leaves behind
    in shared memory, barriers or tensor memory meets the next item on the same CTA."""
    head = (f'extern "C" __global__ void __launch_bounds__({threads}, 1) {name}(const unsigned char *args) {{\n'
            f'  extern __shared__ __align__(16) unsigned char sm[];\n')
    if items is None:
        return head + f'  const int item = blockIdx.x;\n  {statements}\n}}\n'
    return head + f'  for (int item = blockIdx.x; item < {items}; item += gridDim.x) {{\n    {statements}\n    __syncthreads();\n  }}\n}}\n'


def compile_program(source, want_cubin=True):
    """NVRTC: returns the cubin (or PTX) bytes; raises with the log on failure"""
    from cuda.bindings import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"executor.cu", 0, [], [])
    assert err == nvrtc.nvrtcResult.NVRTC_SUCCESS
    opts = [b"--std=c++17", b"--gpu-architecture=sm_100a" if want_cubin else b"--gpu-architecture=compute_100a",
            ("-I" + os.path.join(ROOT, "include")).encode(), ("-I" + CUDA_INCLUDE).encode()]
    err, = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    _, n = nvrtc.nvrtcGetProgramLogSize(prog)
    log = b" " * (n + 8)  # (never a one-byte object: CPython shares those, and the call writes into the buffer)
    nvrtc.nvrtcGetProgramLog(prog, log)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise RuntimeError("NVRTC: " + log.decode(errors="replace")[-4000:])
    if want_cubin:
        _, size = nvrtc.nvrtcGetCUBINSize(prog)
        out = b" " * (size + 8)
        nvrtc.nvrtcGetCUBIN(prog, out)
        out = out[:size]
    else:
        _, size = nvrtc.nvrtcGetPTXSize(prog)
        out = b" " * (size + 8)
        nvrtc.nvrtcGetPTX(prog, out)
        out = out[:size]
    return out


def item_call(lib, p):
    buf = ctypes.create_string_buffer(1024)
    n = lib.mlops_fbla_item_call(ctypes.byref(p), buf, ctypes.c_size_t(1024))
    assert n > 0
    return buf.value.decode()


def run_plan(lib, passes, n, stream, ctas=None):
    """Compiles one kernel per pass and launches them in order on `stream` (a CUDA stream handle): an executor whose only
    dependency rule is 'every item of a pass after every item of the pass before' (stream order). ctas: run every pass
    as a persistent loop on that many CTAs instead of one CTA per item."""
    import numpy as np
    import torch
    from cuda.bindings import driver
    src = POLICY + "".join(kernel_source(f"pass_{i}", passes[i].threads, item_call(lib, passes[i]), None if ctas is None else passes[i].items)
                           for i in range(n))
    cubin = compile_program(src)
    err, module = driver.cuModuleLoadData(cubin)
    assert err == driver.CUresult.CUDA_SUCCESS, err
    keep = []
    for i in range(n):
        p = passes[i]
        err, fn = driver.cuModuleGetFunction(module, f"pass_{i}".encode())
        assert err == driver.CUresult.CUDA_SUCCESS, err
        if p.smem_bytes > 48 * 1024:
            err, = driver.cuFuncSetAttribute(fn, driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, p.smem_bytes)
            assert err == driver.CUresult.CUDA_SUCCESS, err
        blob = torch.from_numpy(np.frombuffer(bytes(p.args.bytes), dtype=np.uint8)[:256].copy()).cuda()  # 16-byte aligned device copy
        keep.append(blob)
        arg = np.array([blob.data_ptr()], dtype=np.uint64)
        params = np.array([arg.ctypes.data], dtype=np.uint64)
        err, = driver.cuLaunchKernel(fn, p.items if ctas is None else min(ctas, p.items), 1, 1, p.threads, 1, 1, p.smem_bytes, stream, params.ctypes.data, 0)
        assert err == driver.CUresult.CUDA_SUCCESS, err
    torch.cuda.synchronize()
    driver.cuModuleUnload(module)
    return keep


def access(lib, passes, n, pass_index, item):
    cnt = lib.mlops_fbla_item_access(passes, n, pass_index, item, None, 0)
    assert cnt >= 0
    arr = (Range * max(cnt, 1))()
    assert lib.mlops_fbla_item_access(passes, n, pass_index, item, arr, cnt) == cnt
    return [arr[i] for i in range(cnt)]
