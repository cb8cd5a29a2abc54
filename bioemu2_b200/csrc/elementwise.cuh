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
                      float eps, int normalize, int silu, const void* __restrict__ x2 = nullptr, int cols1 = 0) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = 1.0f / float(cols);
  for (long long r = warp_global; r < rows; r += warp_stride) {
    // With a second source the row is the concatenation x[r, :cols1] | x2[r, :cols - cols1] (never materialised).
    const int c1 = x2 ? cols1 : cols;
    const uint8_t* xr = static_cast<const uint8_t*>(x) + r * c1 * (long long)(F32IN ? 4 : 2);
    const uint8_t* xr2 = x2 ? static_cast<const uint8_t*>(x2) + r * (cols - c1) * (long long)(F32IN ? 4 : 2) : nullptr;
    uint4 v[4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float f[8];
        if (vi * 8 < c1) load8<F32IN>(xr, vi * 8, f);
        else load8<F32IN>(xr2, vi * 8 - c1, f);
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
          if (silu) {
            a *= sigmoid_fast(a);
            c *= sigmoid_fast(c);
          }
          o[e] = pack_bf16x2(a, c);
        }
        yr[vi] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// The same for narrow rows (cols <= 8 * L, L = 8 or 16 lanes per row): a warp normalises 32 / L rows at a time, one
// 8-channel vector per lane, so that no lane idles on the 64- and 128-channel streams (MSA and pair widths).
template <bool F32IN, int L>
__global__ void __launch_bounds__(256)
layernorm_rows_narrow_kernel(const void* __restrict__ x, __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                             const float* __restrict__ b, long long rows, int cols, float eps, int normalize, int silu) {
  constexpr int RPW = 32 / L;
  const int lane = threadIdx.x & 31;
  const int sub = lane / L, l = lane % L;
  const int nvec = cols >> 3;
  const bool has = l < nvec;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = 1.0f / float(cols);
  float wv[8], bv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    wv[e] = (w && has) ? w[l * 8 + e] : 1.0f;
    bv[e] = (b && has) ? b[l * 8 + e] : 0.0f;
  }
  // every lane runs the same number of iterations: the shuffles below are warp-wide
  for (long long rb = warp_global * RPW; rb < rows; rb += warp_stride * RPW) {
    const long long r = rb + sub;
    const bool act = has && r < rows;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
    if (act) load8<F32IN>(static_cast<const uint8_t*>(x) + r * cols * (long long)(F32IN ? 4 : 2), l * 8, f);
    if (normalize) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) s += f[e];
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * inv;
      float ss = 0.f;
      if (has) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] -= mean;
          ss = fmaf(f[e], f[e], ss);
        }
      }
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss * inv + eps);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = fmaf(f[e] * rstd, wv[e], bv[e]);
      if (silu) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sigmoid_fast(f[e]);
      }
    }
    if (act) store8<false>(y + r * cols, l * 8, f);
  }
}

// Pair initialisation: z[i, j, :] = a[i, :] + c[j, :] (+ extra[i, j, :]) in fp32; one thread per 8 channels,
// cols a multiple of 8.  a and c are tiny and stay in L1/L2: the kernel is the write (and the read of extra).
__global__ void __launch_bounds__(256)
pair_outer_sum_kernel(const float* __restrict__ a, const float* __restrict__ c, const float* __restrict__ extra,
                      float* __restrict__ z, int n_i, int n_j, int cols) {
  const int nvec = cols >> 3;
  const long long total = (long long)n_i * n_j * nvec;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long pair = t / nvec;
    const int v = int(t - pair * nvec);
    const int i = int(pair / n_j), j = int(pair - (long long)i * n_j);
    float fa[8], fc[8];
    load8<true>(a + (long long)i * cols, v * 8, fa);
    load8<true>(c + (long long)j * cols, v * 8, fc);
#pragma unroll
    for (int e = 0; e < 8; ++e) fa[e] += fc[e];
    if (extra) {
      load8<true>(extra + pair * cols, v * 8, fc);
#pragma unroll
      for (int e = 0; e < 8; ++e) fa[e] += fc[e];
    }
    store8<true>(z + pair * cols, v * 8, fa);
  }
}

// out[r, :] = x[r, :] + y[r % period, :]  (x, out fp32 - out may be x; y fp32 or bf16).  period == rows is a plain
// add; a smaller period broadcasts a block of `period` rows over the leading axis.
template <bool YF32>
__global__ void __launch_bounds__(256)
add_rows_kernel(const float* x, const void* __restrict__ y, float* out, long long rows, long long period, int cols) {
  const int nvec = cols >> 3;
  const long long total = rows * nvec;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / nvec;
    const int v = int(t - r * nvec);
    float fx[8], fy[8];
    load8<true>(x + r * cols, v * 8, fx);
    load8<YF32>(static_cast<const uint8_t*>(y) + (r % period) * cols * (long long)(YF32 ? 4 : 2), v * 8, fy);
#pragma unroll
    for (int e = 0; e < 8; ++e) fx[e] += fy[e];
    store8<true>(out + r * cols, v * 8, fx);
  }
}

// h[r, j] = silu(h12[r, j]) * h12[r, H + j]   (bf16 in, bf16 out; H multiple of 8)
__global__ void __launch_bounds__(256)
swiglu_rows_kernel(const __nv_bfloat16* __restrict__ h12, __nv_bfloat16* __restrict__ h, long long rows, int H) {
  const int nvec = H >> 3;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int v = int(i - r * nvec);
    float a[8], b[8];
    load8<false>(h12 + r * 2 * H, v * 8, a);
    load8<false>(h12 + r * 2 * H + H, v * 8, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] * sigmoid_fast(a[e]) * b[e];
    store8<false>(h + r * H, v * 8, a);
  }
}

// y[r,:] = lns * (LN(x[r,:]) * (1 + alpha[r,:]) + beta[r,:]) with alpha/beta columns of a [rows][cw] fp32 tensor
// (adaptive LayerNorm without learned affine); x fp32 or bf16, y bf16.  One warp per row, cols <= 1024.
template <bool F32IN>
__global__ void __launch_bounds__(256)
adaln_rows_kernel(const void* __restrict__ x, const float* __restrict__ cond, int cw, int alpha_col, int beta_col,
                  float lns, __nv_bfloat16* __restrict__ y, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = 1.0f / float(cols);
  for (long long r = warp_global; r < rows; r += warp_stride) {
    const uint8_t* xr = static_cast<const uint8_t*>(x) + r * cols * (long long)(F32IN ? 4 : 2);
    float f[4][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        load8<F32IN>(xr, vi * 8, f[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += f[i][e];
      }
    }
    const float mean = warp_sum(s) * inv;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + i * 32 < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[i][e] -= mean;
          ss = fmaf(f[i][e], f[i][e], ss);
        }
      }
    const float rstd = rsqrtf(warp_sum(ss) * inv + eps);
    const float* cr = cond + r * cw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float al[8], be[8];
        load8<true>(cr + alpha_col, vi * 8, al);
        load8<true>(cr + beta_col, vi * 8, be);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[i][e] = lns * fmaf(f[i][e] * rstd, 1.0f + al[e], be[e]);
        store8<false>(y + r * cols, vi * 8, f[i]);
      }
    }
  }
}

// x[r,:] += gamma[r,:] * h[r,:]  (gamma: columns of a [rows][cw] fp32 tensor; x and h fp32 or bf16)
template <bool XF32, bool HF32>
__global__ void __launch_bounds__(256)
gated_residual_rows_kernel(void* __restrict__ x, const void* __restrict__ h, const float* __restrict__ cond, int cw,
                           int gamma_col, long long rows, int cols) {
  const int nvec = cols >> 3;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int v = int(i - r * nvec);
    float a[8], b[8], g[8];
    uint8_t* xr = static_cast<uint8_t*>(x) + r * cols * (long long)(XF32 ? 4 : 2);
    load8<XF32>(xr, v * 8, a);
    load8<HF32>(static_cast<const uint8_t*>(h) + r * cols * (long long)(HF32 ? 4 : 2), v * 8, b);
    load8<true>(cond + r * cw + gamma_col, v * 8, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = fmaf(g[e], b[e], a[e]);
    store8<XF32>(xr, v * 8, a);
  }
}

// Row softmax of pair-bias logits with the reference's masking convention, one warp per row:
//   w[h][i][j] = softmax_j( mask[i][j] ? logit[h][i][j] : -1e6 )      for i < n_rows, j < n; columns n .. pitch-1 are
//   written as 0.  (n_rows < n when a rank of a context-parallel grid holds only some rows of the weights.)
// The logits arrive in base-2 units (pre-multiplied by log2(e), as the pair-bias projection kernel writes them), bf16;
// the weights leave as bf16.  The row is read three times (maximum, sum, store): it is a few KB and stays in L1/L2.
__global__ void __launch_bounds__(256)
masked_softmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, const uint8_t* __restrict__ mask,
                           __nv_bfloat16* __restrict__ out, int H, int n_rows, int n, int pitch) {
  constexpr float kNegMasked = -1.0e6f * 1.4426950408889634f;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)H * n_rows;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const int nvec = pitch >> 3;
  for (long long r = warp_global; r < rows; r += warp_stride) {
    const int i = int(r % n_rows);
    const __nv_bfloat16* src = logits + r * pitch;
    const uint8_t* mrow = mask + (long long)i * n;
    auto load_masked = [&](int v, float (&x)[8]) {
      load8<false>(src, v * 8, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int j = v * 8 + e;
        x[e] = j < n ? (mrow[j] ? x[e] : kNegMasked) : -INFINITY;
      }
    };
    float mx = -INFINITY;
    for (int v = lane; v < nvec; v += 32) {
      float x[8];
      load_masked(v, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) mx = fmaxf(mx, x[e]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float x[8];
      load_masked(v, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += exp2_approx(x[e] - mx);
    }
    const float inv = 1.0f / warp_sum(sum);
    for (int v = lane; v < nvec; v += 32) {
      float x[8];
      load_masked(v, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = exp2_approx(x[e] - mx) * inv;
      store8<false>(out + r * pitch, v * 8, x);
    }
  }
}

// Gating and re-layout after the pair-weighted average:  og[(s, i)][h*32 + d] = sigmoid(g[(s, i)][h*32 + d]) * o[h][i][s*32 + d]
// (o is what the per-head product  w_h . v_h^T  leaves: token rows, (MSA row, channel) columns).  One thread per 8 channels.
__global__ void __launch_bounds__(256)
pwa_gate_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ og,
                int S, int n, int H) {
  const long long total = (long long)S * n * H * 4;
  const long long o_plane = (long long)n * S * 32;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int d8 = int(t & 3);
    const int h = int((t >> 2) % H);
    const long long si = (t >> 2) / H;          // s * n + i
    const int i = int(si % n);
    const long long s_ = si / n;
    float a[8], b[8];
    load8<false>(o + h * o_plane + ((long long)i * S + s_) * 32, d8 * 8, a);
    load8<false>(g + si * (H * 32) + h * 32, d8 * 8, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] *= sigmoid_fast(b[e]);
    store8<false>(og + si * (H * 32) + h * 32, d8 * 8, a);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// fp32-accurate arithmetic on the bf16 tensor cores: a value x is carried as hi = bf16(x) and lo = bf16(x - hi)
// (16 significant bits together), and a product of two such operands as hi.hi + hi.lo + lo.hi accumulated in fp32.
// With the three pieces laid side by side along K -- (hi | hi | lo) for one operand, (hi | lo | hi) for the other --
// that sum is ONE ordinary K-major product of width 3K, so the GEMM kernel needs no change.
//
// y[r] = split([LayerNorm](x[r])) : x fp32 [rows][cols] -> bf16 [rows][3*cols].  order 0 = (hi | hi | lo), 1 = (hi | lo | hi).
// One warp per row; LayerNorm (fp32, two-pass) only for cols <= 1024.
__global__ void __launch_bounds__(256)
split_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                  const float* __restrict__ b, long long rows, int cols, float eps, int normalize, int order) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  const int nvec = cols >> 3;
  for (long long r = warp_global; r < rows; r += warp_stride) {
    const float* xr = x + r * cols;
    float mean = 0.f, rstd = 1.f;
    if (normalize) {
      float s = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        float f[8];
        load8<true>(xr, v * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += f[e];
      }
      mean = warp_sum(s) / float(cols);
      float ss = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        float f[8];
        load8<true>(xr, v * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e] - mean, f[e] - mean, ss);
      }
      rstd = rsqrtf(warp_sum(ss) / float(cols) + eps);
    }
    __nv_bfloat16* yr = y + r * 3 * (long long)cols;
    for (int v = lane; v < nvec; v += 32) {
      float f[8], hi[8], lo[8];
      load8<true>(xr, v * 8, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (normalize) {
          f[e] = (f[e] - mean) * rstd;
          if (w) f[e] *= w[v * 8 + e];
          if (b) f[e] += b[v * 8 + e];
        }
        hi[e] = __bfloat162float(__float2bfloat16_rn(f[e]));
        lo[e] = f[e] - hi[e];
      }
      store8<false>(yr, v * 8, hi);
      store8<false>(yr + cols, v * 8, order ? lo : hi);
      store8<false>(yr + 2 * cols, v * 8, order ? hi : lo);
    }
  }
}

// fp32 gating: out[r][c] = a[r][c] * act(b[r][c]) [* (rowmask[r] != 0)], a and b given with their own row pitches.
// mode 0: a * sigmoid(b) (gated projections); mode 1: silu(a) * b (SwiGLU); mode 2: a alone (row masking only).
// Accurate exponentials, no approximations.
__global__ void __launch_bounds__(256)
gate_rows_f32_kernel(const float* __restrict__ a, long long a_pitch, const float* __restrict__ b, long long b_pitch,
                     const uint8_t* __restrict__ rowmask, float* __restrict__ out, long long rows, int cols, int mode) {
  const int nvec = cols >> 2;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int v = int(i - r * nvec);
    const float4 av = *reinterpret_cast<const float4*>(a + r * a_pitch + v * 4);
    const float4 bv = *reinterpret_cast<const float4*>(b + r * b_pitch + v * 4);
    const float keep = (rowmask == nullptr || rowmask[r]) ? 1.f : 0.f;
    float x[4] = {av.x, av.y, av.z, av.w}, g[4] = {bv.x, bv.y, bv.z, bv.w}, o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = keep * (mode == 0 ? x[e] / (1.f + expf(-g[e])) : mode == 1 ? x[e] / (1.f + expf(-x[e])) * g[e] : x[e]);
    *reinterpret_cast<float4*>(out + r * cols + v * 4) = make_float4(o[0], o[1], o[2], o[3]);
  }
}

// fp32 softmax over keys of attention logits with an additive bias and the reference's key mask:
//   p[g][q][k] = softmax_k( keymask[g / mask_div][k] ? s[g][q][k] + bias[g_bias][q][k] : -1e6 ),   in place in s,
// g_bias = (g / (H * bias_div)) * H + g % H  (the bias of a batch item is shared by its `bias_div` copies).
__global__ void __launch_bounds__(256)
softmax_bias_f32_kernel(float* __restrict__ s, const float* __restrict__ bias, const uint8_t* __restrict__ keymask,
                        long long groups, int n, int H, int bias_div, int mask_div_heads) {
  const int lane = threadIdx.x & 31;
  const long long rows = groups * n;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = warp_global; r < rows; r += warp_stride) {
    const long long g = r / n;
    const int q = int(r - g * n);
    const long long gb = (g / ((long long)H * bias_div)) * H + g % H;
    float* sr = s + r * n;
    const float* br = bias ? bias + (gb * n + q) * (long long)n : nullptr;
    const uint8_t* mr = keymask + (g / mask_div_heads) * n;
    float mx = -INFINITY;
    for (int k = lane; k < n; k += 32) {
      const float v = mr[k] ? sr[k] + (br ? br[k] : 0.f) : -1.0e6f;
      sr[k] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int k = lane; k < n; k += 32) {
      const float e = expf(sr[k] - mx);
      sr[k] = e;
      sum += e;
    }
    const float inv = 1.f / warp_sum(sum);
    for (int k = lane; k < n; k += 32) sr[k] *= inv;
  }
}

}  // namespace b200
