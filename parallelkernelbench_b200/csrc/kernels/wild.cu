// Small compute kernels of the project-derived workloads (each is the local half of a fused exchange + compute op).
#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

// ------------------------------------------------------------------------------------------------
// DISCO contraction on the sphere: y[bc, row, p] = sum_e val[e] * x[bc, lat[e], (lon[e] + p * pscale) mod nlon_in]
// for the entries e of sparse row `row` = (kernel index, output latitude). One thread per (bc, row, p); the
// reference loops over p with a sparse bmm and a roll of the whole input per step
// (reference: reference/62_torchharmonics_spherical_convolution.py:42-69).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
disco_contract_kernel(const float* __restrict__ x, const int* __restrict__ row_ptr, const int* __restrict__ col,
                      const float* __restrict__ val, float* __restrict__ y, long long bc, int rows, int nlat_in,
                      int nlon_in, int nlon_out, int pscale) {
  const long long total = bc * rows * nlon_out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i % nlon_out);
    const long long t = i / nlon_out;
    const int row = (int)(t % rows);
    const long long b = t / rows;
    const float* xb = x + b * nlat_in * nlon_in;
    float acc = 0.f;
    for (int e = row_ptr[row]; e < row_ptr[row + 1]; ++e) {
      const int c = col[e];
      const int lat = c / nlon_in;
      int lon = c - lat * nlon_in + p * pscale;
      lon %= nlon_in;
      acc += val[e] * xb[lat * nlon_in + lon];
    }
    y[i] = acc;
  }
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_disco_contract(const void* x, const void* row_ptr, const void* col, const void* val, void* y,
                                  long long bc, int rows, int nlat_in, int nlon_in, int nlon_out, void* stream) {
  PKB_CHECK_ARG(bc >= 1 && rows >= 1 && nlat_in >= 1 && nlon_in >= 1 && nlon_out >= 1 && nlon_in % nlon_out == 0,
                "bad DISCO shape (nlon_in must be a multiple of nlon_out)");
  const long long total = bc * rows * nlon_out;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  disco_contract_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), static_cast<const int*>(row_ptr), static_cast<const int*>(col),
      static_cast<const float*>(val), static_cast<float*>(y), bc, rows, nlat_in, nlon_in, nlon_out, nlon_in / nlon_out);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
