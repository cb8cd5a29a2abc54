// Sliding-window attention with pair bias for the atom transformer: a query window of W atoms attends to the Hk keys
// centred on it (context = (Hk - W) / 2 atoms on either side, zero rows beyond the ends of the sequence).
//
// The work is small and oddly shaped for the tensor cores (32 x 128 scores per window and head, head dim 32): for
// ~4,000 atoms it is a fraction of a GFLOP per sample, while the pair features that feed the bias are tens of MB.
// So the two kernels here are plain fp32 CUDA-core kernels and the arithmetic of the core - scores, softmax and the
// weighted sum - is exact fp32, as in the reference's autocast-free block.
//
//   window_bias_kernel       bias[b][w][h][i][j] = proj_z(LayerNorm(z[b][w][i][j][:]))[h], c_z / 4 lanes per pair
//   window_attention_kernel  one CTA per (sample, window): K and V rows of the window staged in shared memory as bf16,
//                            one thread per (head, query), online softmax over the keys in chunks of 8
#pragma once
#include "elementwise.cuh"

namespace b200 {

struct WindowBiasParams {
  const void* z;       // [pairs][c_z], fp32 or bf16
  const float* ln_w;   // [c_z]
  const float* ln_b;   // [c_z] or nullptr
  const float* w_z;    // [heads][c_z]
  float* bias;         // [pairs / (W*Hk)][heads][W*Hk]
  long long pairs;     // B * NW * W * Hk
  int window_pairs;    // W * Hk
  int c_z, heads;
  float eps;
};

constexpr int kWindowMaxHeads = 16;

// A group of LPR lanes (a power of two >= c_z / 4) shares one pair: each lane holds four channels, the LayerNorm
// statistics and the per-head dot products are reduced across the group with shuffles, so a warp's loads cover
// 32 / LPR consecutive rows (contiguous memory) instead of 32 rows a stride apart.
template <bool F32>
__global__ void __launch_bounds__(256)
window_bias_kernel(WindowBiasParams p, int lpr) {
  const int lane = threadIdx.x & 31;
  const int sub = lane / lpr, l = lane % lpr;
  const int rpw = 32 / lpr;
  const bool has = l * 4 < p.c_z;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * (blockDim.x >> 5);
  float g[4] = {0.f, 0.f, 0.f, 0.f}, bt[4] = {0.f, 0.f, 0.f, 0.f};
  if (has) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      g[e] = p.ln_w[l * 4 + e];
      bt[e] = p.ln_b ? p.ln_b[l * 4 + e] : 0.f;
    }
  }
  const float inv = 1.0f / float(p.c_z);
  // every lane runs the same number of iterations: the shuffles are warp-wide
  for (long long rb = warp_global * rpw; rb < p.pairs; rb += warp_stride * rpw) {
    const long long t = rb + sub;
    const bool act = has && t < p.pairs;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (act) {
      if (F32) {
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.z) + t * p.c_z + l * 4);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
      } else {
        const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.z) + t * p.c_z + l * 4);
        x[0] = bf16lo(v.x); x[1] = bf16hi(v.x); x[2] = bf16lo(v.y); x[3] = bf16hi(v.y);
      }
    }
    float s = (x[0] + x[1]) + (x[2] + x[3]);
    for (int o = lpr >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * inv;
    float ss = 0.f;
    if (has) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x[e] -= mean;
        ss = fmaf(x[e], x[e], ss);
      }
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * inv + p.eps);
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = has ? fmaf(x[e] * rstd, g[e], bt[e]) : 0.f;
    const long long win = t / p.window_pairs;
    const int ij = int(t - win * p.window_pairs);
    float* dst = p.bias + win * p.heads * p.window_pairs + ij;
    for (int h = 0; h < p.heads; ++h) {
      float acc = 0.f;
      if (has) {
        const float* wr = p.w_z + h * p.c_z + l * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc = fmaf(y[e], __ldg(wr + e), acc);
      }
      for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (l == (h % lpr) && t < p.pairs) dst[(long long)h * p.window_pairs] = acc;
    }
  }
}

struct WindowAttnParams {
  const __nv_bfloat16* qkv;   // [BM][L][3 * c_s]: q (bias added) | k | v, L = NW * W atoms
  const __nv_bfloat16* gate;  // [BM][L][c_s] gate logits
  const float* bias;          // [B][NW][heads][W][Hk]
  const uint8_t* mask;        // [B][L], non-zero = valid atom
  __nv_bfloat16* out;         // [BM][L][c_s] = sigmoid(gate) * attention output
  int NW, W, Hk, heads, M;
  float scale;                // 1 / sqrt(head dim)
};

constexpr float kWindowMasked = -1e6f;  // the reference REPLACES masked logits by -inf = -1e6 (masked_fill_)

template <int DH>
__global__ void __launch_bounds__(256)
window_attention_kernel(WindowAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const int c_s = p.heads * DH;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vs = Ks + (size_t)p.Hk * c_s;
  uint8_t* kvalid = reinterpret_cast<uint8_t*>(Vs + (size_t)p.Hk * c_s);

  const int f = blockIdx.x;
  const int bm = f / p.NW, w = f - bm * p.NW, b = bm / p.M;
  const int L = p.NW * p.W;
  const int a0 = w * p.W - (p.Hk - p.W) / 2;  // atom index of key 0 (may be negative)
  const long long item = (long long)bm * L;

  // stage the window's K and V rows (zero rows outside the sequence, as the zero-padded unfold gives)
  const int vec_per_row = c_s >> 3;
  for (int idx = threadIdx.x; idx < p.Hk * vec_per_row; idx += blockDim.x) {
    const int j = idx / vec_per_row, v = idx - j * vec_per_row;
    const int a = a0 + j;
    uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
    if (a >= 0 && a < L) {
      const __nv_bfloat16* src = p.qkv + (item + a) * 3 * c_s + c_s + v * 8;
      kk = *reinterpret_cast<const uint4*>(src);
      vv = *reinterpret_cast<const uint4*>(src + c_s);
    }
    reinterpret_cast<uint4*>(Ks)[idx] = kk;
    reinterpret_cast<uint4*>(Vs)[idx] = vv;
  }
  for (int j = threadIdx.x; j < p.Hk; j += blockDim.x) {
    const int a = a0 + j;
    kvalid[j] = (a >= 0 && a < L && p.mask[(long long)b * L + a]) ? 1 : 0;
  }
  __syncthreads();

  const int h = threadIdx.x / p.W, i = threadIdx.x - h * p.W;
  if (h >= p.heads) return;
  const long long atom = item + w * p.W + i;
  float q[DH], o[DH];
  {
    const __nv_bfloat16* qs = p.qkv + atom * 3 * c_s + h * DH;
#pragma unroll
    for (int d = 0; d < DH; d += 8) {
      float x[8];
      load8<false>(qs, d, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) q[d + e] = x[e] * p.scale;
    }
  }
#pragma unroll
  for (int d = 0; d < DH; ++d) o[d] = 0.f;
  const float* brow = p.bias + ((((long long)b * p.NW + w) * p.heads + h) * p.W + i) * p.Hk;
  float m = -INFINITY, l = 0.f;
  for (int j0 = 0; j0 < p.Hk; j0 += 8) {
    float s[8];
    const float4 b0 = *reinterpret_cast<const float4*>(brow + j0), b1 = *reinterpret_cast<const float4*>(brow + j0 + 4);
    const float bj[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    float cmax = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const __nv_bfloat16* kr = Ks + (size_t)(j0 + jj) * c_s + h * DH;
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < DH; d += 8) {
        float x[8];
        load8<false>(kr, d, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = fmaf(q[d + e], x[e], acc);
      }
      s[jj] = kvalid[j0 + jj] ? acc + bj[jj] : kWindowMasked;
      cmax = fmaxf(cmax, s[jj]);
    }
    const float m_new = fmaxf(m, cmax);
    const float corr = __expf(m - m_new);  // 0 on the first chunk (m = -inf)
    l *= corr;
#pragma unroll
    for (int d = 0; d < DH; ++d) o[d] *= corr;
    m = m_new;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const float pj = __expf(s[jj] - m);
      l += pj;
      const __nv_bfloat16* vr = Vs + (size_t)(j0 + jj) * c_s + h * DH;
#pragma unroll
      for (int d = 0; d < DH; d += 8) {
        float x[8];
        load8<false>(vr, d, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[d + e] = fmaf(pj, x[e], o[d + e]);
      }
    }
  }
  const float inv_l = 1.0f / l;
  const __nv_bfloat16* gs = p.gate + atom * c_s + h * DH;
  __nv_bfloat16* dst = p.out + atom * c_s + h * DH;
#pragma unroll
  for (int d = 0; d < DH; d += 8) {
    float g[8], y[8];
    load8<false>(gs, d, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = o[d + e] * inv_l / (1.0f + __expf(-g[e]));
    store8<false>(dst, d, y);
  }
}

}  // namespace b200
