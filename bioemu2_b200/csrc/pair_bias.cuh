// Pair bias projection (see the comment above the kernel).
#pragma once
#include "row_tile.cuh"

namespace b200 {

// -------------------------------------------------------------------------------------------------
// Pair bias: zb[h][i][j] = scale * proj_z(LN_z(z[i, j, :]))[h] for up to 16 heads, bf16, row pitch Nk.
// A tile is 128 consecutive j of one row i: producers LayerNorm the rows into an MMA operand, one
// 128 x 16 x 128 product per tile, lanes = pairs so every head's row is stored coalesced.
//   warps 0-3 epilogue, warps 4-11 producers, warp 12 control.
struct PairBiasParams {
  const void* z;        // pair-tensor slab, fp32 or bf16, 128 channels per pair
  const float* ln_w;
  const float* ln_b;    // nullptr: LayerNorm without bias
  __nv_bfloat16* zb;    // [H][lines][pitch]
  int n_lines, n_pos;   // slab geometry: pair (line, pos) at z + line*z_line_stride + pos*z_pos_stride (bytes);
  long long z_line_stride, z_pos_stride;  // swap the strides to get the bias of the transposed pair tensor
  long long out_plane, out_pitch;         // zb[h*out_plane + line*out_pitch + pos] (elements)
  int H;
  int num_tiles;        // n_lines * ceil(n_pos/128)
  float scale;          // log2(e)
  float eps;
};

namespace pair_bias {
constexpr uint32_t W_OFF = 0;                   // 16 rows x 256 B as two 16-row halves of 128 B rows: 2 x 2 KB
constexpr uint32_t X_OFF = 4096;                // 2 stages x 32 KB
constexpr uint32_t BAR_OFF = X_OFF + 2 * kOperandTile;
constexpr uint32_t SMEM_BYTES = BAR_OFF + 128 + 1024;
constexpr int THREADS = 416;
}  // namespace pair_bias

template <bool F32>
__global__ void __launch_bounds__(416, 1)
pair_bias_kernel(const __grid_constant__ CUtensorMap tmW, PairBiasParams p) {
  using namespace pair_bias;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = w_full + 1;
  uint64_t* x_empty = x_full + 2;
  uint64_t* acc_full = x_empty + 2;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_row = (p.n_pos + 127) >> 7;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&x_full[i], 256);
      mbar_init(&x_empty[i], 1);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tmap(&tmW);
  }
  if (warp == 12) tmem_alloc(tmem_slot, 32);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 12) {
    // The whole warp walks the tile loop and waits on the barriers; one elected lane issues the products and the
    // commits (a converged warp issues a tcgen05.mma several times faster than a lone thread of a diverged one).
    const bool leader = elect_one();
    if (leader) {
      mbar_arrive_expect_tx(w_full, 4096);
      tma_load_2d(smem + W_OFF, &tmW, w_full, 0, 0);
      tma_load_2d(smem + W_OFF + 2048, &tmW, w_full, 64, 0);
    }
    __syncwarp();
    mbar_wait(w_full, 0, 80);
    constexpr uint32_t idesc = make_idesc_bf16(128, 16);
    const uint32_t w_s = smem_u32(smem + W_OFF);
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_full[s], (it >> 1) & 1, 81);
      mbar_wait(&acc_empty[s], ((it >> 1) & 1) ^ 1, 82);
      tc_fence_after_sync();
      const uint32_t x_s = smem_u32(smem + X_OFF + s * kOperandTile);
      const uint32_t x_lo = desc_lo(x_s), w_lo = desc_lo(w_s);
      if (leader) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss2(tmem_base + s * 16, x_lo + (k >> 2) * (kOperandHalf >> 4) + (k & 3) * 2, kDescHiSw128,
                        w_lo + (k >> 2) * (2048 >> 4) + (k & 3) * 2, kDescHiSw128, idesc, k > 0);
        umma_commit(&x_empty[s]);
        umma_commit(&acc_full[s]);
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    const int pt = threadIdx.x - 128;
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_w, p.ln_b, pt, gamma, beta);
    RowTile<256> regs;
    const long long pos_stride = p.z_pos_stride, line_stride = p.z_line_stride;
    auto load_tile = [&](int tile) {
      const int i = tile / tiles_per_row;
      const int j0 = (tile - i * tiles_per_row) << 7;
      const uint8_t* base = static_cast<const uint8_t*>(p.z) + i * line_stride;
      regs.template load<F32, true>(
          pt, [&](int r) -> const void* { return (j0 + r) < p.n_pos ? base + (j0 + r) * pos_stride : nullptr; },
          gamma, beta, p.eps);
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_empty[s], ((it >> 1) & 1) ^ 1, 83);
      regs.store_operand(pt, smem + X_OFF + s * kOperandTile);
      fence_proxy_async_smem();
      mbar_arrive(&x_full[s]);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int i = tile / tiles_per_row;
      const int j = ((tile - i * tiles_per_row) << 7) + warp * 32 + lane;
      const int acc = it & 1;
      mbar_wait(&acc_full[acc], (it >> 1) & 1, 84);
      tc_fence_after_sync();
      uint32_t v[16];
      tmem_ld_32x16(tmem_addr(tmem_base, warp * 32, acc * 16), v);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
      if (j < p.n_pos) {
#pragma unroll
        for (int h = 0; h < 16; ++h)
          if (h < p.H) p.zb[h * p.out_plane + i * p.out_pitch + j] = __float2bfloat16(__uint_as_float(v[h]) * p.scale);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) {
    __syncwarp();
    tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace b200
