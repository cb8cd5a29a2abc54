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
//
// The 4-head triangle bias  b[h][line][pos] = log2(e) * (LN(x) . w_b[h])  is one more projection of the same
// normalised rows, so the kernel produces it too and the pair tensor is read once per triangle attention instead of
// twice.  There is no free TMEM column and 2 KB of shared memory left: the bias product (128 x 16 x 128) lands in q's
// first 16 columns as soon as the epilogue has read them, and its weight operand is the 8 rows that hold the 4 heads,
// read twice by a descriptor with a row-group stride of zero (heads 8..15 are copies that nobody reads).
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
  __nv_bfloat16* tri_bias;  // [4][lines][bias_pitch], or nullptr: the triangle bias is not produced here
  long long bias_plane;     // elements between heads
  int bias_pitch;
  float bias_scale;         // log2(e)
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
constexpr uint32_t WB_OFF = STAGE_OFF + 2 * kOperandHalf;  // bias weights: 8 rows x 128 B per 64-channel half, 2 x 1 KB
constexpr uint32_t SMEM_BYTES = WB_OFF + 2048;       // exactly the 227 KB an SM offers: the base must be 1024-aligned
constexpr int THREADS = 416;
}  // namespace triatt_proj

template <bool F32>
__global__ void __launch_bounds__(416, 1)
triatt_proj_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQKG,
                   const __grid_constant__ CUtensorMap tmVT, const __grid_constant__ CUtensorMap tmWB,
                   TriAttProjParams p) {
  using namespace triatt_proj;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need the alignment; there is no room to round up
    if (threadIdx.x == 0 && atomicCAS(&g_dev_status, 0, kDevWaitTimeout | (99 << 8)) == 0) {
      int* hp = g_host_status_ptr;
      if (hp) {
        *reinterpret_cast<volatile int*>(hp) = kDevWaitTimeout | (99 << 8);
        __threadfence_system();
      }
    }
    return;
  }
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = w_full + 1;     // [2] count 256
  uint64_t* x_empty = x_full + 2;    // [2] commit
  uint64_t* acc_full = x_empty + 2;  // [2] group A, group B
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* q0_drained = acc_empty + 2;  // count 128: q's first columns have been read, the bias product may land there
  uint64_t* bias_full = q0_drained + 1;  // commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bias_full + 1);
  const bool fuse_bias = p.tri_bias != nullptr;
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
    mbar_init(q0_drained, 128);
    mbar_init(bias_full, 1);
    fence_mbar_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmQKG);
    prefetch_tmap(&tmVT);
    prefetch_tmap(&tmWB);
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
      mbar_arrive_expect_tx(w_full, 4 * kOperandTile + (fuse_bias ? 2048 : 0));
      for (int mt = 0; mt < 4; ++mt)
        for (int h = 0; h < 2; ++h)
          tma_load_2d(smem + W_OFF + mt * kOperandTile + h * kOperandHalf, &tmW, w_full, h * 64, mt * 128);
      if (fuse_bias) {
        tma_load_2d(smem + WB_OFF, &tmWB, w_full, 0, 0);
        tma_load_2d(smem + WB_OFF + 1024, &tmWB, w_full, 64, 0);
      }
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
        if (!fuse_bias) umma_commit(&x_empty[s]);
      }
      __syncwarp();
      if (fuse_bias) {  // bias[pair][head] into q's columns 0..15, once the epilogue has taken q's first chunk out
        mbar_wait(q0_drained, it & 1, 98);
        tc_fence_after_sync();
        if (leader) {
          constexpr uint32_t idesc_b = make_idesc_bf16(128, 16);
          constexpr uint32_t kDescHiSw128Sbo0 = (1u << 14) | (2u << 29);  // both 8-row groups read the same 8 rows
          const uint32_t x_lo = desc_lo(x_s), wb_lo = desc_lo(smem_u32(smem + WB_OFF));
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_bf16_ss2(tmem_base, x_lo + (k >> 2) * (kOperandHalf >> 4) + (k & 3) * 2, kDescHiSw128,
                          wb_lo + (k >> 2) * (1024 >> 4) + (k & 3) * 2, kDescHiSw128Sbo0, idesc_b, k > 0);
          umma_commit(bias_full);
          umma_commit(&x_empty[s]);
        }
        __syncwarp();
      }
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
        if (c == 0 && fuse_bias) {  // q's columns 0..31 are in registers: the bias product may overwrite them
          tc_fence_before_sync();
          mbar_arrive(q0_drained);
        }
        if (c == 7) {  // q, k read: the next tile's group A products may start; g, V^T must have landed
          if (fuse_bias) {  // ... after the bias that sits in q's columns has been stored: head h of pair r
            mbar_wait(bias_full, it & 1, 99);
            tc_fence_after_sync();
            uint32_t bv[16];
            tmem_ld_32x16(tmem_addr(tmem_base, warp * 32, 0), bv);
            tmem_ld_wait();
            if (pos0 + r < p.n_pos) {
              __nv_bfloat16* dstb = p.tri_bias + (long long)line * p.bias_pitch + pos0 + r;
#pragma unroll
              for (int h = 0; h < 4; ++h) dstb[h * p.bias_plane] = __float2bfloat16(__uint_as_float(bv[h]) * p.bias_scale);
            }
          }
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
