// Batched C[b] = scale * A[b] * B[b]^T with both operands K-major bf16, fp32
// accumulation in tensor memory and bf16 output.
//
// This is the per-channel contraction of triangle multiplication
// (t[d][i][j] = sum_k a[d][i][k] * b[d][j][k]) and the MSA-depth contraction of
// the outer product mean.  Persistent kernel, one CTA per SM:
//   warp 0      TMA producer   (A and B K-slabs of 64 through a shared-memory ring)
//   warp 1      MMA issuer     (tcgen05.mma 128 x BN x 16, two accumulator buffers in TMEM)
//   warps 2..5  epilogue       (TMEM -> registers -> bf16 -> global)
#pragma once
#include "row_tile.cuh"

namespace b200 {

struct BmmParams {
  void* C;                   // bf16, or fp32 when out_f32
  long long c_batch_stride;  // elements
  int ldc;                   // elements
  int m_valid, n_valid;      // rows / columns of C that exist (n_valid % 8 == 0)
  int tiles_m, tiles_n, batch;
  int k_blocks;              // K / 64, rounded up (TMA zero-fills the tail)
  float scale;
  const float* scale_ptr;    // optional per-batch device scalar multiplied into scale
  const float* bias;         // optional per-column bias added after scaling
  int out_f32;
  // Outer-product store: with opm_ntok > 0, C row r = (i, c) and column q = (j, d) (c, d < 32) go to
  // C[((i * opm_ntok + j) * 32 + c) * 32 + d]: every pair (i, j) gets its 32x32 outer product contiguous.
  int opm_ntok;
  // Residual and transposed pair store (output projection of triangle attention): with residual != nullptr
  // the value read from it at the destination offset is added; with remap_n > 0 row r = line * remap_n + pos
  // (line < remap_m) is stored as row pos * remap_m + line.
  const void* residual;
  int remap_n, remap_m;
  // Bulk output: the scaled (+ bias) tile leaves through 16 KB staging tiles ([128 rows][128 B]: 32 fp32 or 64
  // bf16 columns) and the C tensor map, 1 = stored, 2 = added into C (the residual is C itself, which the
  // epilogue then never reads).
  int tma_c;
  int a_shared;              // 1: every batch item multiplies the same A (the A tensor map has a single batch slice)
};

template <int BN>
struct BmmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr uint32_t OUT_OFFSET = BAR_OFFSET + 1024;        // two [128 rows][128 B] tiles for bulk output
  static constexpr uint32_t SMEM_BYTES = OUT_OFFSET + 2 * 16384 + 1024;  // + alignment slack
  static constexpr int THREADS = 192;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
bmm_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
              const __grid_constant__ CUtensorMap tmC, BmmParams p) {
  using Cfg = BmmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFFSET);
  uint64_t* empty = full + Cfg::STAGES;
  uint64_t* acc_full = empty + Cfg::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.tma_c) prefetch_tmap(&tmC);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        const int rem = tile - b * tiles_per_batch;
        const int tm = rem / p.tiles_n;
        const int tn = rem - tm * p.tiles_n;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          mbar_wait(&empty[stage], phase ^ 1, 1);
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          tma_load_3d(sa, &tmA, &full[stage], kb * 64, tm * 128, p.a_shared ? 0 : b);
          tma_load_3d(sa + Cfg::A_BYTES, &tmB, &full[stage], kb * 64, tn * BN, b);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the tile and K loops and waits on the barriers; one elected lane issues the products and
    // the commits (a converged warp issues a tcgen05.mma several times faster than a lone thread of a diverged one).
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(128, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        mbar_wait(&acc_empty[acc], ((it >> 1) & 1) ^ 1, 2);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          mbar_wait(&full[stage], phase, 3);
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
          const uint32_t a_lo = desc_lo(sa), b_lo = desc_lo(sb);
          if (leader) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16_ss2(d_tmem, a_lo + 2 * k, kDescHiSw128, b_lo + 2 * k, kDescHiSw128, idesc, (kb | k) != 0);
            umma_commit(&empty[stage]);
          }
          __syncwarp();
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (leader) umma_commit(&acc_full[acc]);
        __syncwarp();
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter .. +31
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int b = tile / tiles_per_batch;
      const int rem = tile - b * tiles_per_batch;
      const int tm = rem / p.tiles_n;
      const int tn = rem - tm * p.tiles_n;
      const int acc = it & 1;
      mbar_wait(&acc_full[acc], (it >> 1) & 1, 4);
      tc_fence_after_sync();
      const int row = tm * 128 + quarter * 32 + lane;
      const float scale = p.scale_ptr ? p.scale * p.scale_ptr[b] : p.scale;
      if (p.tma_c) {
        // 32 columns at a time into one of two swizzled staging tiles; warp 2's first lane sends each tile off.
        const int r = quarter * 32 + lane;
        const bool leader = threadIdx.x == 64;
        int c1 = tm * 128, c2 = b;  // tensor map {column, row, batch}, or {column, line, pos} when remapped
        if (p.remap_n > 0) {
          c1 = (tm * 128) / p.remap_n;
          c2 = tm * 128 - c1 * p.remap_n;
        }
        const int cps = p.out_f32 ? 1 : 2;  // 32-column chunks per staging tile
        uint32_t va[32], vb[32];
        tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, acc * BN), va);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t(&v)[32] = (c & 1) ? vb : va;
          const int st = p.out_f32 ? c : (c >> 1);  // staging tile number within the output tile
          uint8_t* stage = smem + Cfg::OUT_OFFSET + (st & 1) * 16384;
          if (p.out_f32 || (c & 1) == 0) {
            if (leader) tma_store_wait_read1();  // the store that last used this staging tile has read it
            named_bar_sync(1, 128);
          }
          tmem_ld_wait();
          if (c + 1 < BN / 32) {
            tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, acc * BN + (c + 1) * 32), (c & 1) ? va : vb);
          } else {
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[acc]);
          }
          const int col0 = tn * BN + c * 32;
          if (p.out_f32) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              float4 x;
              x.x = __uint_as_float(v[g * 4 + 0]) * scale;
              x.y = __uint_as_float(v[g * 4 + 1]) * scale;
              x.z = __uint_as_float(v[g * 4 + 2]) * scale;
              x.w = __uint_as_float(v[g * 4 + 3]) * scale;
              if (p.bias && col0 + g * 4 < p.n_valid) {  // n_valid % 8 == 0: a group of four is inside or outside
                const float4 bv = *reinterpret_cast<const float4*>(p.bias + col0 + g * 4);
                x.x += bv.x; x.y += bv.y; x.z += bv.z; x.w += bv.w;
              }
              *reinterpret_cast<float4*>(stage + sw128_offset(r, g)) = x;
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float x[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[g * 8 + e]) * scale;
              if (p.bias && col0 + g * 8 < p.n_valid) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] += p.bias[col0 + g * 8 + e];
              }
              *reinterpret_cast<uint4*>(stage + sw128_offset(r, (c & 1) * 4 + g)) = make_uint4(
                  pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
            }
          }
          if (p.out_f32 || (c & 1) == 1) {
            const int tcol0 = tn * BN + st * 32 * cps;
            fence_proxy_async_smem();
            named_bar_sync(1, 128);
            if (leader && tcol0 < p.n_valid) {
              if (p.tma_c == 2)
                tma_reduce_add_3d(&tmC, stage, tcol0, c1, c2);
              else
                tma_store_3d(&tmC, stage, tcol0, c1, c2);
              tma_store_commit();
            }
          }
        }
        continue;
      }
      const size_t esz = p.out_f32 ? 4 : 2;
      uint8_t* cbase = static_cast<uint8_t*>(p.C) + (long long)b * p.c_batch_stride * esz;
      // 32 columns at a time; the next chunk's TMEM load and (when a residual is added) its residual row
      // segment are requested before the current chunk is processed.
      const uint8_t* rbase = p.residual ? static_cast<const uint8_t*>(p.residual) + (long long)b * p.c_batch_stride * esz
                                        : nullptr;
      auto chunk_off = [&](int c) -> long long {  // element offset of (row, first column of chunk c)
        const int col0 = tn * BN + c * 32;
        if (p.opm_ntok > 0) return (((long long)(row >> 5) * p.opm_ntok + (col0 >> 5)) * 32 + (row & 31)) * 32;
        if (p.remap_n > 0) return ((long long)(row % p.remap_n) * p.remap_m + row / p.remap_n) * p.ldc + col0;
        return (long long)row * p.ldc + col0;
      };
      auto load_res = [&](int c, float (&rz)[32]) {
        const long long off0 = chunk_off(c);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float t8[8];
          const bool ok = rbase && row < p.m_valid && (tn * BN + c * 32 + g * 8) < p.n_valid;
          if (ok) {
            if (p.out_f32)
              load8<true>(rbase + (off0 + g * 8) * 4, 0, t8);
            else
              load8<false>(rbase + (off0 + g * 8) * 2, 0, t8);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) rz[g * 8 + e] = ok ? t8[e] : 0.f;
        }
      };
      uint32_t va[32], vb[32];
      float ra[32], rb[32];
      tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, acc * BN), va);
      load_res(0, ra);
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t(&v)[32] = (c & 1) ? vb : va;
        float(&rz)[32] = (c & 1) ? rb : ra;
        tmem_ld_wait();
        if (c + 1 < BN / 32) {
          tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, acc * BN + (c + 1) * 32), (c & 1) ? va : vb);
          load_res(c + 1, (c & 1) ? ra : rb);
        }
        if (row < p.m_valid) {
          const int col0 = tn * BN + c * 32;
          const long long off0 = chunk_off(c);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col < p.n_valid) {
              float x[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) x[e] = fmaf(__uint_as_float(v[g * 8 + e]), scale, rz[g * 8 + e]);
              if (p.bias) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] += p.bias[col + e];
              }
              if (p.out_f32)
                store8<true>(cbase + (off0 + g * 8) * 4, 0, x);
              else
                store8<false>(cbase + (off0 + g * 8) * 2, 0, x);
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  if (p.tma_c && threadIdx.x == 64) tma_store_wait0();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200
