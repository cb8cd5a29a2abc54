// HBM-bound row kernels: 128-bit loads and stores, one warp per row, fp32 statistics.
#pragma once
#include "row_tile.cuh"

namespace b200 {

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// y[r,:] = LN(x[r,:]) * w + b for rows of `cols` <= 1024 channels (multiple of 8); x fp32 or bf16, y bf16.
// With normalize == 0 the rows are only converted to bf16.
template <bool F32IN>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const void* __restrict__ x, __nv_bfloat16* __restrict__ y,
                      const float* __restrict__ w, const float* __restrict__ b, long long rows, int cols,
                      float eps, int normalize) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = 1.0f / float(cols);
  for (long long r = warp_global; r < rows; r += warp_stride) {
    const uint8_t* xr = static_cast<const uint8_t*>(x) + r * cols * (long long)(F32IN ? 4 : 2);
    uint4 v[4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float f[8];
        load8<F32IN>(xr, vi * 8, f);
        v[i] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                          pack_bf16x2(f[6], f[7]));
#pragma unroll
        for (int e = 0; e < 8; ++e) s += f[e];
      } else {
        v[i] = make_uint4(0, 0, 0, 0);
      }
    }
    if (!normalize) {
      uint4* yr0 = reinterpret_cast<uint4*>(y + r * cols);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (lane + i * 32 < nvec) yr0[lane + i * 32] = v[i];
      continue;
    }
    const float mean = warp_sum(s) * inv;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (lane + i * 32 < nvec) {
        const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a = bf16lo(u[e]) - mean, c = bf16hi(u[e]) - mean;
          ss = fmaf(a, a, fmaf(c, c, ss));
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(ss) * inv + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + r * cols);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c0 = vi * 8 + e * 2;
          float a = (bf16lo(u[e]) - mean) * rstd, c = (bf16hi(u[e]) - mean) * rstd;
          if (w) {
            a *= w[c0];
            c *= w[c0 + 1];
          }
          if (b) {
            a += b[c0];
            c += b[c0 + 1];
          }
          o[e] = pack_bf16x2(a, c);
        }
        yr[vi] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

}  // namespace b200
