// Outer product mean, projection stage: m'[s, i, :] = mask * proj_ab(LN(m[s, i, :])) for c_in = 64,
// c_hidden = 32, written transposed -- aT[(i, c)][s], bT[(j, d)][s] (bf16, pitch Sp) -- so that the
// contraction over the MSA depth s is a plain K-major A.B^T for bmm_nt_kernel, whose outer-product
// store then lays each pair's 32x32 block out contiguously for the output projection.
//
// A tile is one token i and 128 consecutive MSA rows s.
//   warps 0-3  epilogue (TMEM lane = s; mask; transposed bf16 stores)
//   warps 4-7  producers (load rows, LayerNorm over 64 channels, write the A operand)
//   warp  8    control (TMA of proj_ab, MMA issue)
#pragma once
#include "row_tile.cuh"

namespace b200 {

struct OpmProjParams {
  const void* m;         // [S][N][64] fp32 or bf16 (one batch element)
  const uint8_t* mask;   // [S][N] (mask_s_stride = N) or [N] (mask_s_stride = 0); non-zero = valid
  long long mask_s_stride;
  const float* ln_w;
  const float* ln_b;
  __nv_bfloat16* aT;     // [N*32][Sp]
  __nv_bfloat16* bT;
  int S, N, Sp;
  int num_tiles;         // N * ceil(S/128)
  float eps;
};

namespace opm_proj {
constexpr uint32_t W_OFF = 0;                      // 64 rows x 128 B
constexpr uint32_t X_OFF = 8192;                   // 2 stages x 16 KB
constexpr uint32_t BAR_OFF = X_OFF + 2 * kOperandHalf;
constexpr uint32_t SMEM_BYTES = BAR_OFF + 128 + 1024;
constexpr int THREADS = 288;
}  // namespace opm_proj

__device__ __forceinline__ float group8_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

template <bool F32>
__global__ void __launch_bounds__(288, 1)
opm_proj_kernel(const __grid_constant__ CUtensorMap tmW, OpmProjParams p) {
  using namespace opm_proj;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = w_full + 1;     // [2] count 128
  uint64_t* x_empty = x_full + 2;    // [2] commit
  uint64_t* acc_full = x_empty + 2;  // [2] commit
  uint64_t* acc_empty = acc_full + 2;  // [2] count 128
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_tok = (p.S + 127) >> 7;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&x_full[i], 128);
      mbar_init(&x_empty[i], 1);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tmap(&tmW);
  }
  if (warp == 8) tmem_alloc(tmem_slot, 128);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // the whole warp waits on the barriers, one elected lane issues
    const bool leader = elect_one();
    if (leader) {
      mbar_arrive_expect_tx(w_full, 8192);
      tma_load_2d(smem + W_OFF, &tmW, w_full, 0, 0);
    }
    __syncwarp();
    mbar_wait(w_full, 0, 50);
    constexpr uint32_t idesc = make_idesc_bf16(128, 64);
    const uint32_t w_s = smem_u32(smem + W_OFF);
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_full[s], (it >> 1) & 1, 51);
      mbar_wait(&acc_empty[s], ((it >> 1) & 1) ^ 1, 52);
      tc_fence_after_sync();
      const uint32_t x_s = smem_u32(smem + X_OFF + s * kOperandHalf);
      const uint32_t x_lo = desc_lo(x_s), w_lo = desc_lo(w_s);
      if (leader) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss2(tmem_base + s * 64, x_lo + 2 * k, kDescHiSw128, w_lo + 2 * k, kDescHiSw128, idesc, k > 0);
        umma_commit(&x_empty[s]);
        umma_commit(&acc_full[s]);
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    // producers: 8 threads per row (8 channels each), 16 rows per pass, 8 passes
    const int pt = threadIdx.x - 128;
    const int c8 = pt & 7;
    const int rbase = pt >> 3;
    float gamma[8], beta[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      gamma[i] = p.ln_w[c8 * 8 + i];
      beta[i] = p.ln_b[c8 * 8 + i];
    }
    uint4 held[8];
    auto load_tile = [&](int tile) {
      const int tok = tile / tiles_per_tok;
      const int s0 = (tile - tok * tiles_per_tok) << 7;
      float x[8][8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int s = s0 + q * 16 + rbase;
        if (s < p.S) {
          load8<F32>(static_cast<const uint8_t*>(p.m) + ((long long)s * p.N + tok) * 64 * zbytes<F32>(), c8 * 8, x[q]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[q][i] = 0.f;
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += x[q][i];
        const float mean = group8_sum(sum) * (1.0f / 64);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[q][i] -= mean;
          ss = fmaf(x[q][i], x[q][i], ss);
        }
        const float rstd = rsqrtf(group8_sum(ss) * (1.0f / 64) + p.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[q][i] = fmaf(x[q][i] * rstd, gamma[i], beta[i]);
        held[q] = make_uint4(pack_bf16x2(x[q][0], x[q][1]), pack_bf16x2(x[q][2], x[q][3]),
                             pack_bf16x2(x[q][4], x[q][5]), pack_bf16x2(x[q][6], x[q][7]));
      }
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_empty[s], ((it >> 1) & 1) ^ 1, 53);
      uint8_t* dst = smem + X_OFF + s * kOperandHalf;
#pragma unroll
      for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(dst + sw128_offset(q * 16 + rbase, c8)) = held[q];
      fence_proxy_async_smem();
      mbar_arrive(&x_full[s]);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    // epilogue: lane = MSA row s of the tile
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int tok = tile / tiles_per_tok;
      const int s = ((tile - tok * tiles_per_tok) << 7) + warp * 32 + lane;
      const int acc = it & 1;
      const bool in_range = s < p.S;
      const bool valid = in_range && p.mask[(long long)s * p.mask_s_stride + tok] != 0;
      mbar_wait(&acc_full[acc], (it >> 1) & 1, 54);
      tc_fence_after_sync();
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, acc * 64 + half * 32), v);
        tmem_ld_wait();
        if (in_range) {
          __nv_bfloat16* dst = (half ? p.bT : p.aT) + (long long)tok * 32 * p.Sp + s;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            dst[(long long)c * p.Sp] = __float2bfloat16(valid ? __uint_as_float(v[c]) : 0.f);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem_base, 128);
  }
}

// Number of MSA rows with at least one valid token -> 1 / max(count, 1).  One block.
__global__ void opm_inv_row_count_kernel(const uint8_t* mask, int S, int N, float* inv_out) {
  __shared__ int count;
  if (threadIdx.x == 0) count = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int local = 0;
  for (int s = warp; s < S; s += nwarps) {
    bool any = false;
    for (int i = lane; i < N; i += 32) any |= mask[(long long)s * N + i] != 0;
    if (__any_sync(0xffffffffu, any)) ++local;
  }
  if (lane == 0 && local) atomicAdd(&count, local);
  __syncthreads();
  if (threadIdx.x == 0) *inv_out = 1.0f / float(count > 0 ? count : 1);
}

}  // namespace b200
