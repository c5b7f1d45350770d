"""Example solution for the op `tp_rmsnorm` that brings its own CUDA kernels.

The hidden dimension is sharded over the ranks: every rank sums the squares of its columns per row (kernel 1), the row sums
are added over the ranks with one small all-reduce on the symmetric heap, and kernel 2 scales the rows. The kernels are
compiled for sm_100a on first use by `compile_cuda_module` (cached on disk; concurrent ranks wait on a file lock) and
called through ctypes with raw pointers and the current stream. CPU ranks take the PyTorch path."""
import ctypes

import torch

_SRC = r'''
#include <cuda_bf16.h>

// one warp per row: fp32 sum of squares of a bf16 row
__global__ void row_sumsq(const __nv_bfloat16* x, float* ss, int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float acc = 0.f;
  for (int c = lane; c < cols; c += 32) { const float v = __bfloat162float(x[(long long)row * cols + c]); acc += v * v; }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) ss[row] = acc;
}

__global__ void row_scale(const __nv_bfloat16* x, const __nv_bfloat16* w, const float* ss, __nv_bfloat16* y, int rows, int cols,
                          float inv_n, float eps) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int row = (int)(i / cols), c = (int)(i - (long long)row * cols);
  const float r = rsqrtf(ss[row] * inv_n + eps);
  y[i] = __float2bfloat16_rn(__bfloat162float(w[c]) * (__bfloat162float(x[i]) * r));
}

extern "C" int ex_row_sumsq(const void* x, void* ss, int rows, int cols, void* stream) {
  row_sumsq<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                        static_cast<float*>(ss), rows, cols);
  return (int)cudaGetLastError();
}
extern "C" int ex_row_scale(const void* x, const void* w, const void* ss, void* y, int rows, int cols, float inv_n, float eps,
                            void* stream) {
  const long long n = (long long)rows * cols;
  row_scale<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const float*>(ss),
      static_cast<__nv_bfloat16*>(y), rows, cols, inv_n, eps);
  return (int)cudaGetLastError();
}
'''
_lib = None


def _kernels():
    global _lib
    if _lib is None:
        from parallelkernelbench_b200.utils.cuda_ext import compile_cuda_module

        _lib = compile_cuda_module(_SRC, name="example_tp_rmsnorm")
    return _lib


def solution(rc, x, w, eps):
    rows, cols = x.shape
    if not x.is_cuda or x.dtype != torch.bfloat16:
        ss = rc.comm.all_reduce(x.float().pow(2).sum(-1, keepdim=True).contiguous())
        return (w.float() * (x.float() * torch.rsqrt(ss / (cols * rc.world) + eps))).to(x.dtype)
    lib, stream = _kernels(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x, w = x.contiguous(), w.contiguous()
    ss = torch.empty(rows, dtype=torch.float32, device=x.device)
    assert lib.ex_row_sumsq(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(ss.data_ptr()), rows, cols, stream) == 0
    ss = rc.comm.all_reduce(ss)                       # rows * 4 bytes: the no-barrier exchange for small messages
    y = torch.empty_like(x)
    assert lib.ex_row_scale(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(ss.data_ptr()),
                            ctypes.c_void_p(y.data_ptr()), rows, cols, ctypes.c_float(1.0 / (cols * rc.world)),
                            ctypes.c_float(eps), stream) == 0
    return y
