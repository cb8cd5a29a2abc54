// Triangle attention, projection stage: h = LN(x);  q | k | g = h Wq^T, h Wk^T, sigmoid(h Wg^T + b_g)  (pair-major,
// bf16, row pitch 384) and V^T = Wv h^T (channel-major per line, bf16, pitch Nk), the layouts the flash
// core reads.  x is the pair tensor for the starting node and its transpose for the ending node: a tile
// is 128 consecutive `pos` on one `line`, pair (line, pos) = z[line][pos] or z[pos][line].
//
//   warps 0-3   epilogue: q, k (lane = pair), then g (lane = pair) and V^T (lane = channel)
//   warps 4-11  producers: load rows, LayerNorm, write the shared operand tile (A for q/k/g, B for V^T)
//   warp  12    control: TMA of the weights (resident), MMA issue
// TMEM: q 0..127, k 128..255 (group A), g 256..383, V^T 384..511 (group B); each group has its own
// full/empty barriers so the next tile's products start while the other group is being stored.
#pragma once
#include "row_tile.cuh"

namespace b200 {

struct TriAttProjParams {
  const void* z;         // pair-tensor slab, fp32 or bf16: pair (line, pos) at z + line*z_line_stride + pos*z_pos_stride
  const float* ln_w;
  const float* ln_b;
  const float* g_bias;   // [128]
  __nv_bfloat16* qkg;    // [lines][n_pos][384]
  __nv_bfloat16* vT;     // [lines][128][Nk]
  int n_lines, n_pos, Nk;
  long long z_line_stride, z_pos_stride;  // bytes; starting node: line = row, ending node: line = column
  int num_tiles;         // n_lines * ceil(n_pos/128)
  float eps;
};

namespace triatt_proj {
constexpr uint32_t W_OFF = 0;                        // Wq, Wk, Wg, Wv: 4 x 32 KB
constexpr uint32_t X_OFF = 4 * kOperandTile;         // 2 stages x 32 KB
constexpr uint32_t GB_OFF = X_OFF + 2 * kOperandTile;  // gate bias, 512 B
constexpr uint32_t BAR_OFF = GB_OFF + 512;
constexpr uint32_t STAGE_OFF = GB_OFF + 1024;        // two 16 KB output tiles [128 rows][128 B] for the TMA stores
constexpr uint32_t SMEM_BYTES = STAGE_OFF + 2 * kOperandHalf + 1024;
constexpr int THREADS = 416;
}  // namespace triatt_proj

template <bool F32>
__global__ void __launch_bounds__(416, 1)
triatt_proj_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQKG,
                   const __grid_constant__ CUtensorMap tmVT, TriAttProjParams p) {
  using namespace triatt_proj;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = w_full + 1;     // [2] count 256
  uint64_t* x_empty = x_full + 2;    // [2] commit
  uint64_t* acc_full = x_empty + 2;  // [2] group A, group B
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* gb_s = reinterpret_cast<float*>(smem + GB_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_line = (p.n_pos + 127) >> 7;

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
    prefetch_tmap(&tmQKG);
    prefetch_tmap(&tmVT);
  }
  if (threadIdx.x < 128) gb_s[threadIdx.x] = p.g_bias[threadIdx.x];
  if (warp == 12) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 12) {
    // The whole warp walks the tile loop and waits on the barriers; one elected lane issues the products and the
    // commits (a converged warp issues a tcgen05.mma several times faster than a lone thread of a diverged one).
    const bool leader = elect_one();
    if (leader) {
      mbar_arrive_expect_tx(w_full, 4 * kOperandTile);
      for (int mt = 0; mt < 4; ++mt)
        for (int h = 0; h < 2; ++h)
          tma_load_2d(smem + W_OFF + mt * kOperandTile + h * kOperandHalf, &tmW, w_full, h * 64, mt * 128);
    }
    __syncwarp();
    mbar_wait(w_full, 0, 90);
    constexpr uint32_t idesc = make_idesc_bf16(128, 128);
    const uint32_t w_s = smem_u32(smem + W_OFF);
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_full[s], (it >> 1) & 1, 91);
      const uint32_t x_s = smem_u32(smem + X_OFF + s * kOperandTile);
      mbar_wait(&acc_empty[0], (it & 1) ^ 1, 92);
      tc_fence_after_sync();
      if (leader) {
        umma_k128(tmem_base + 0, x_s, w_s + 0 * kOperandTile, idesc, false);    // q  [pair][ch]
        umma_k128(tmem_base + 128, x_s, w_s + 1 * kOperandTile, idesc, false);  // k
        umma_commit(&acc_full[0]);
      }
      __syncwarp();
      mbar_wait(&acc_empty[1], (it & 1) ^ 1, 93);
      tc_fence_after_sync();
      if (leader) {
        umma_k128(tmem_base + 256, x_s, w_s + 2 * kOperandTile, idesc, false);  // g  [pair][ch]
        umma_k128(tmem_base + 384, w_s + 3 * kOperandTile, x_s, idesc, false);  // V^T [ch][pair]
        umma_commit(&acc_full[1]);
        umma_commit(&x_empty[s]);
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    const int pt = threadIdx.x - 128;
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_w, p.ln_b, pt, gamma, beta);
    const long long pos_stride = p.z_pos_stride, line_stride = p.z_line_stride;
    RowTile<256> regs;
    auto load_tile = [&](int tile) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      const uint8_t* base = static_cast<const uint8_t*>(p.z) + line * line_stride;
      regs.template load<F32, true>(
          pt,
          [&](int r) -> const void* {
            const int pos = pos0 + r;
            return pos < p.n_pos ? base + pos * pos_stride : nullptr;
          },
          gamma, beta, p.eps);
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_empty[s], ((it >> 1) & 1) ^ 1, 94);
      regs.store_operand(pt, smem + X_OFF + s * kOperandTile);
      fence_proxy_async_smem();
      mbar_arrive(&x_full[s]);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    const int r = warp * 32 + lane;  // TMEM lane: pair of the tile for q/k/g, channel for V^T
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      // The 512 accumulator columns leave as eight [128 rows][64 values] bf16 tiles through two swizzled
      // staging tiles and TMA stores: q, k (4 tiles) and g + bias (2 tiles) with lane = pair into the pair-major
      // rows, V^T (2 tiles) with lane = channel into the line's channel-major plane.  TMEM is read 32 columns
      // at a time with the next chunk's load in flight.
      uint32_t va[32], vb[32];
      const bool leader = threadIdx.x == 0;
      mbar_wait(&acc_full[0], it & 1, 95);
      tc_fence_after_sync();
      tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, 0), va);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint32_t(&v)[32] = (c & 1) ? vb : va;
        uint8_t* stage = smem + STAGE_OFF + ((c >> 1) & 1) * kOperandHalf;
        tmem_ld_wait();
        if (c == 7) {  // q, k read: the next tile's group A products may start; g, V^T must have landed
          tc_fence_before_sync();
          mbar_arrive(&acc_empty[0]);
          mbar_wait(&acc_full[1], it & 1, 96);
          tc_fence_after_sync();
        }
        if (c < 15) {
          tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, (c + 1) * 32), (c & 1) ? va : vb);
        } else {
          tc_fence_before_sync();
          mbar_arrive(&acc_empty[1]);
        }
        uint4 packed[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float y[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(v[g * 8 + e]);
          if (c >= 8 && c < 12) {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = sigmoid_fast(y[e] + gb_s[(c - 8) * 32 + g * 8 + e]);  // the gate leaves activated
          }
          packed[g] = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                 pack_bf16x2(y[6], y[7]));
        }
        if ((c & 1) == 0) {  // the store that last used this staging tile has finished reading it (the wait hides
          if (leader) tma_store_wait_read1();  // behind the conversion above)
          named_bar_sync(1, 128);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(stage + sw128_offset(r, (c & 1) * 4 + g)) = packed[g];
        if (c & 1) {
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (leader) {
            if (c < 12)
              tma_store_3d(&tmQKG, stage, (c >> 1) * 64, pos0, line);
            else
              tma_store_3d(&tmVT, stage, pos0 + ((c >> 1) - 6) * 64, 0, line);
            tma_store_commit();
          }
        }
      }
    }
  }

  if (threadIdx.x == 0) tma_store_wait0();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200
