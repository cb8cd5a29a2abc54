// Sliding-window attention with pair bias for the atom transformer: a query window of W atoms attends to the Hk keys
// centred on it (context = (Hk - W) / 2 atoms on either side, zero rows beyond the ends of the sequence).
//
// The work is small and oddly shaped for the tensor cores (32 x 128 scores per window and head, head dim 32): for
// ~4,000 atoms it is a fraction of a GFLOP per sample, while the pair features that feed the bias are tens of MB.
// So the two kernels here are plain fp32 CUDA-core kernels and the arithmetic of the core - scores, softmax and the
// weighted sum - is exact fp32, as in the reference's autocast-free block.
//
//   window_bias_kernel       bias[b][w][h][i][j] = proj_z(LayerNorm(z[b][w][i][j][:]))[h], one thread per pair
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

template <bool F32>
__global__ void __launch_bounds__(256)
window_bias_kernel(WindowBiasParams p) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < p.pairs; t += (long long)gridDim.x * blockDim.x) {
    const uint8_t* row = static_cast<const uint8_t*>(p.z) + t * p.c_z * (long long)(F32 ? 4 : 2);
    auto ld = [&](int c) -> float {
      return F32 ? reinterpret_cast<const float*>(row)[c]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(row)[c]);
    };
    float s = 0.f;
    for (int c = 0; c < p.c_z; ++c) s += ld(c);
    const float mean = s / float(p.c_z);
    float ss = 0.f;
    for (int c = 0; c < p.c_z; ++c) {
      const float d = ld(c) - mean;
      ss = fmaf(d, d, ss);
    }
    const float rstd = rsqrtf(ss / float(p.c_z) + p.eps);
    float acc[kWindowMaxHeads];
#pragma unroll
    for (int h = 0; h < kWindowMaxHeads; ++h) acc[h] = 0.f;
    for (int c = 0; c < p.c_z; ++c) {
      const float y = fmaf((ld(c) - mean) * rstd, __ldg(p.ln_w + c), p.ln_b ? __ldg(p.ln_b + c) : 0.f);
#pragma unroll
      for (int h = 0; h < kWindowMaxHeads; ++h)
        if (h < p.heads) acc[h] = fmaf(y, __ldg(p.w_z + h * p.c_z + c), acc[h]);
    }
    const long long win = t / p.window_pairs;
    const int ij = int(t - win * p.window_pairs);
    float* dst = p.bias + win * p.heads * p.window_pairs + ij;
#pragma unroll
    for (int h = 0; h < kWindowMaxHeads; ++h)
      if (h < p.heads) dst[(long long)h * p.window_pairs] = acc[h];
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
