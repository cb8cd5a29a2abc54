// Building blocks shared by the kernels that walk the pair tensor in tiles of
// 128 pair rows x 128 channels.  A group of NT threads (128 or 256) loads the rows
// with wide loads (16 threads per row, 8 channels each), applies LayerNorm in fp32
// as the data arrives and keeps the bf16 result in registers until the shared-memory
// stage is free; it is then written as a K-major, 128-byte-swizzled MMA operand.
//
// The pair tensor ("z stream") is either fp32 -- what the reference keeps under bf16
// autocast, since the residual adds promote to fp32 -- or bf16.
#pragma once
#include "umma.cuh"

namespace b200 {

constexpr int kD = 128;                   // pair channels (c_z)
constexpr uint32_t kOperandHalf = 16384;  // bytes of one 128-row x 64-channel operand half
constexpr uint32_t kOperandTile = 32768;  // 128 rows x 128 channels bf16

__device__ __forceinline__ void ld_global_v8(const float* p, float (&x)[8]) {
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3]), "=f"(x[4]), "=f"(x[5]), "=f"(x[6]), "=f"(x[7])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ void st_global_v8(float* p, const float (&x)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(x[0]), "f"(x[1]), "f"(x[2]),
               "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7])
               : "memory");
}

// 8 consecutive channels of a row of the z stream -> fp32 registers.  Plain (coherent) loads: several
// kernels update the stream in place, so nothing goes through the read-only path.
template <bool F32>
__device__ __forceinline__ void load8(const void* row, int c0, float (&x)[8]) {
  if (F32) {
    ld_global_v8(static_cast<const float*>(row) + c0, x);
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(row) + c0);
    x[0] = bf16lo(v.x); x[1] = bf16hi(v.x); x[2] = bf16lo(v.y); x[3] = bf16hi(v.y);
    x[4] = bf16lo(v.z); x[5] = bf16hi(v.z); x[6] = bf16lo(v.w); x[7] = bf16hi(v.w);
  }
}
template <bool F32>
__device__ __forceinline__ void store8(void* row, int c0, const float (&x)[8]) {
  if (F32) {
    st_global_v8(static_cast<float*>(row) + c0, x);
  } else {
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(row) + c0) =
        make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
  }
}
template <bool F32>
__host__ __device__ constexpr size_t zbytes() { return F32 ? 4 : 2; }

__device__ __forceinline__ float group16_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// One thread's share of a 128-row tile: rows q*(NT/16) + pt/16 (q = 0..RPT-1), channels 8*(pt%16)..+7,
// held as packed bf16 after the (optional) LayerNorm.
template <int NT>
struct RowTile {
  static constexpr int RPT = 128 * 16 / NT;  // rows per thread
  static constexpr int RSTEP = NT / 16;
  uint4 v[RPT];

  // row_ptr(r) -> address of channel 0 of tile row r (elements of the z stream), or nullptr if absent.
  // LS: rows normalised in lock step by the one-pass packed form (8 where the kernel has registers to spare);
  // LS = 1 selects the register-tight two-pass form.
  template <bool F32, bool NORM, int LS = 8, class RowPtr>
  __device__ __forceinline__ void load(int pt, RowPtr row_ptr, const float (&gamma)[8], const float (&beta)[8],
                                       float eps, float raw_scale = 1.0f) {
    const int c0 = (pt & 15) * 8;
    const int rbase = pt >> 4;
#pragma unroll
    for (int q0 = 0; q0 < RPT; q0 += 8) {
      float x[8][8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const void* src = row_ptr((q0 + q) * RSTEP + rbase);
        if (src) {
          load8<F32>(src, c0, x[q]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[q][i] = 0.f;
        }
      }
      if (NORM && LS == 1) {
        // Register-tight form for kernels compiled at 96 registers: rows one after the other, two-pass variance.
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float sm = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) sm += x[q][i];
          const float mean = group16_sum(sm) * (1.0f / kD);
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x[q][i] -= mean;
            ss = fmaf(x[q][i], x[q][i], ss);
          }
          const float rstd = rsqrtf(group16_sum(ss) * (1.0f / kD) + eps);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[q][i] = fmaf(x[q][i] * rstd, gamma[i], beta[i]);
          v[q0 + q] = make_uint4(pack_bf16x2(x[q][0], x[q][1]), pack_bf16x2(x[q][2], x[q][3]),
                                 pack_bf16x2(x[q][4], x[q][5]), pack_bf16x2(x[q][6], x[q][7]));
        }
      } else if (NORM) {
        // One pass: row sum and sum of squares together (packed fp32x2 arithmetic, one 16-lane butterfly for the
        // pair), then y = x * (rstd * gamma) + (beta - mean * rstd * gamma).  LS rows go through the butterfly
        // in lock step.  (Sum of squares minus squared mean in fp32: the relative error of the variance is
        // about 1e-7 * (1 + mean^2 / var), far below bf16 resolution for any realistic row.)
#pragma unroll
        for (int qb = 0; qb < 8; qb += LS) {
          float s1[LS], s2[LS];
#pragma unroll
          for (int q = 0; q < LS; ++q) {
            const float* xr = x[qb + q];
            float a0 = xr[0], a1 = xr[1], b0, b1;
            add_f32x2(a0, a1, xr[2], xr[3]);
            add_f32x2(a0, a1, xr[4], xr[5]);
            add_f32x2(a0, a1, xr[6], xr[7]);
            mul_f32x2(b0 = xr[0], b1 = xr[1], xr[0], xr[1]);
            fma_f32x2(b0, b1, xr[2], xr[3], xr[2], xr[3], b0, b1);
            fma_f32x2(b0, b1, xr[4], xr[5], xr[4], xr[5], b0, b1);
            fma_f32x2(b0, b1, xr[6], xr[7], xr[6], xr[7], b0, b1);
            s1[q] = a0 + a1;
            s2[q] = b0 + b1;
          }
#pragma unroll
          for (int off = 8; off > 0; off >>= 1) {
#pragma unroll
            for (int q = 0; q < LS; ++q) {
              const float o1 = __shfl_xor_sync(0xffffffffu, s1[q], off);
              const float o2 = __shfl_xor_sync(0xffffffffu, s2[q], off);
              add_f32x2(s1[q], s2[q], o1, o2);
            }
          }
#pragma unroll
          for (int q = 0; q < LS; ++q) {
            float* xr = x[qb + q];
            const float mean = s1[q] * (1.0f / kD);
            const float var = fmaxf(fmaf(-mean, mean, s2[q] * (1.0f / kD)), 0.f);
            const float rstd = rsqrtf(var + eps);
            const float nmr = -mean * rstd;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
              float g0 = gamma[i], g1 = gamma[i + 1], b0, b1;
              fma_f32x2(b0, b1, g0, g1, nmr, nmr, beta[i], beta[i + 1]);  // beta - mean * rstd * gamma
              mul_f32x2(g0, g1, rstd, rstd);                              // rstd * gamma
              fma_f32x2(xr[i], xr[i + 1], xr[i], xr[i + 1], g0, g1, b0, b1);
            }
            v[q0 + qb + q] = make_uint4(pack_bf16x2(xr[0], xr[1]), pack_bf16x2(xr[2], xr[3]), pack_bf16x2(xr[4], xr[5]),
                                        pack_bf16x2(xr[6], xr[7]));
          }
        }
      } else {  // no LayerNorm: the rows are only scaled by raw_scale (a power of two keeps them exact)
#pragma unroll
        for (int q = 0; q < 8; ++q) {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[q][i] *= raw_scale;
          v[q0 + q] = make_uint4(pack_bf16x2(x[q][0], x[q][1]), pack_bf16x2(x[q][2], x[q][3]),
                                 pack_bf16x2(x[q][4], x[q][5]), pack_bf16x2(x[q][6], x[q][7]));
        }
      }
    }
  }

  // Write the held rows into the operand tile at `dst` (shared memory, 1024-byte aligned).
  __device__ __forceinline__ void store_operand(int pt, uint8_t* dst) const {
    const int c16 = pt & 15;
    const int rbase = pt >> 4;
    uint8_t* half = dst + (c16 >> 3) * kOperandHalf;
#pragma unroll
    for (int q = 0; q < RPT; ++q)
      *reinterpret_cast<uint4*>(half + sw128_offset(q * RSTEP + rbase, c16 & 7)) = v[q];
  }
};

// scale multiplies the LayerNorm output; a power of two keeps the result a bit-exact multiple.
__device__ __forceinline__ void load_gamma_beta(const float* w, const float* b, int pt, float (&gamma)[8],
                                                float (&beta)[8], float scale = 1.0f) {
  const int c0 = (pt & 15) * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    gamma[i] = (w ? w[c0 + i] : 1.0f) * scale;
    beta[i] = (b ? b[c0 + i] : 0.0f) * scale;
  }
}

// Issue the 8 K-steps of a 128 x N x 128 product: A and B operand tiles are 128-swizzled halves.
__device__ __forceinline__ void umma_k128(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, uint32_t idesc,
                                          bool accumulate_first) {
  const uint32_t a_lo = desc_lo(a_smem), b_lo = desc_lo(b_smem);  // one add per operand per step in the loop
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = (k >> 2) * (kOperandHalf >> 4) + (k & 3) * 2;
    umma_bf16_ss2(d_tmem, a_lo + off, kDescHiSw128, b_lo + off, kDescHiSw128, idesc, (accumulate_first || k > 0) ? 1u : 0u);
  }
}

}  // namespace b200
