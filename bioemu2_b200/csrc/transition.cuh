// Pair transition: out = fc3( silu(fc1(h)) * fc2(h) ) [+ x],  h = LN(x) (or x), dim 128 -> hidden 512 -> 128.
//
// One persistent CTA per SM walks tiles of 128 pair rows.  The hidden axis is processed in 8 chunks of
// 64: GEMM1 writes [fc1 chunk | fc2 chunk] (128 x 128) to one of two TMEM buffers, a warpgroup turns it
// into the bf16 SwiGLU product in shared memory (K-major operand), GEMM2 accumulates it against the
// matching 64-wide slice of fc3 into the output accumulator (two of them, so the final store of a tile
// overlaps the next tile's GEMMs).  The hidden activations never leave the SM.
//
// The GEMM1 input is halved (exactly), so with a' = fc1/2, b' = fc2/2 the SwiGLU product is
// silu(a) b = 2 (u + u tanh(a')) with u = a' b': one MUFU and two FMA-pipe operations per hidden element; the
// factor 2 is applied to the output accumulator.  The output leaves through swizzled [128 rows][64 B] staging
// tiles and TMA: added into x in place when the residual is wanted and out aliases x, stored otherwise.
//
//   warps 0-3   SwiGLU epilogue of even chunks
//   warps 4-7   SwiGLU epilogue of odd chunks
//   warps 8-15  producers: load rows, LayerNorm, write the GEMM1 A operand; they also send out the previous
//               tile's output accumulator (warps 8-11 channels 0-63, warps 12-15 channels 64-127), so the
//               SwiGLU groups never leave the chunk pipeline
//   warp  16    GEMM1 issuer
//   warp  17    TMA loader for the [fc1|fc2] chunks
//   warp  18    GEMM2 issuer
//   warp  19    TMA loader for the fc3 slices
#pragma once
#include "row_tile.cuh"

namespace b200 {

struct TransitionParams {
  const void* x;           // [rows][128] fp32 or bf16
  void* out;               // [rows][128] same dtype, may alias x
  const float* ln_w;       // nullptr with use_norm == 0
  const float* ln_b;
  long long rows;
  int num_tiles;
  int use_norm;
  int add_residual;
  float eps;
};

namespace transition {
constexpr int CHUNKS = 8;  // hidden 512 = 8 x 64
constexpr int WS = 3;      // weight chunk stages: the chunk loads come from L2 and need two chunk times to land
constexpr uint32_t X_OFF = 0;                            // 32 KB (A of GEMM1)
constexpr uint32_t W1_OFF = X_OFF + kOperandTile;        // WS stages x 32 KB ([fc1|fc2] chunk, 128 rows x 128 K)
constexpr uint32_t W3_OFF = W1_OFF + WS * kOperandTile;  // WS stages x 16 KB (fc3 slice, 128 rows x 64 K)
constexpr uint32_t H_OFF = W3_OFF + WS * kOperandHalf;   // 2 buffers x 16 KB (A of GEMM2, 128 rows x 64 K)
constexpr uint32_t BAR_OFF = H_OFF + 2 * kOperandHalf;
constexpr uint32_t STAGE_OFF = BAR_OFF + 1024;           // per output half-group one 8 KB output tile
constexpr uint32_t SMEM_BYTES = STAGE_OFF + 2 * 8192 + 1024;
constexpr int THREADS = 640;
}  // namespace transition

template <bool F32>
__global__ void __launch_bounds__(640, 1)
transition_kernel(const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmW3,
                  const __grid_constant__ CUtensorMap tmO, TransitionParams p) {
  using namespace transition;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = bars;            // count 256
  uint64_t* x_empty = bars + 1;       // commit
  uint64_t* w1_full = bars + 2;       // [WS] TMA
  uint64_t* w1_empty = bars + 5;      // [WS] commit
  uint64_t* w3_full = bars + 8;       // [WS] TMA
  uint64_t* w3_empty = bars + 11;     // [WS] commit
  uint64_t* d1_full = bars + 14;      // [2] commit
  uint64_t* d1_empty = bars + 16;     // [2] count 128
  uint64_t* h_full = bars + 18;       // [2] count 128
  uint64_t* h_empty = bars + 20;      // [2] commit
  uint64_t* out_full = bars + 22;     // [2] commit
  uint64_t* out_empty = bars + 24;    // [2] count 256
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 256);
    mbar_init(x_empty, 1);
    for (int i = 0; i < WS; ++i) {
      mbar_init(&w1_full[i], 1);
      mbar_init(&w1_empty[i], 1);
      mbar_init(&w3_full[i], 1);
      mbar_init(&w3_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&d1_full[i], 1);
      mbar_init(&d1_empty[i], 128);
      mbar_init(&h_full[i], 128);
      mbar_init(&h_empty[i], 1);
      mbar_init(&out_full[i], 1);
      mbar_init(&out_empty[i], 256);
    }
    fence_mbar_init();
    prefetch_tmap(&tmW1);
    prefetch_tmap(&tmW3);
    prefetch_tmap(&tmO);
  }
  if (warp == 16) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: D1[b] at b*128 (fc1 chunk 0..63, fc2 chunk 64..127); OUT[o] at 256 + o*128.

  int my_tiles = 0;
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) ++my_tiles;
  const int total_chunks = my_tiles * CHUNKS;
  // A global chunk counter g = it*8 + c drives the rings: depth 2 (stage g&1, use g>>1) for the TMEM and H
  // buffers, depth WS (stage g%WS, use g/WS) for the weight chunks.

  if (warp == 17) {
    // ------------------------------------------------------------------ [fc1|fc2] chunk loader (TMA)
    if (lane == 0) {
      for (int g = 0; g < total_chunks; ++g) {
        const int c = g & 7, s = g % WS;
        mbar_wait(&w1_empty[s], ((g / WS) & 1) ^ 1, 30);
        mbar_arrive_expect_tx(&w1_full[s], kOperandTile);
        tma_load_2d(smem + W1_OFF + s * kOperandTile, &tmW1, &w1_full[s], 0, c * 128);
        tma_load_2d(smem + W1_OFF + s * kOperandTile + kOperandHalf, &tmW1, &w1_full[s], 64, c * 128);
      }
    }
  } else if (warp == 19) {
    // ------------------------------------------------------------------ fc3 slice loader (TMA)
    if (lane == 0) {
      for (int g = 0; g < total_chunks; ++g) {
        const int c = g & 7, s = g % WS;
        mbar_wait(&w3_empty[s], ((g / WS) & 1) ^ 1, 31);
        mbar_arrive_expect_tx(&w3_full[s], kOperandHalf);
        tma_load_2d(smem + W3_OFF + s * kOperandHalf, &tmW3, &w3_full[s], c * 64, 0);
      }
    }
  } else if (warp == 16) {
    // ------------------------------------------------------------------ GEMM1 issuer
    // (both issuers: the whole warp walks the chunk loop and waits on the barriers, one elected lane issues)
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      for (int g = 0; g < total_chunks; ++g) {
        const int c = g & 7, b = g & 1, it = g >> 3, ws = g % WS;
        if (c == 0) mbar_wait(x_full, it & 1, 35);
        mbar_wait(&w1_full[ws], (g / WS) & 1, 36);
        mbar_wait(&d1_empty[b], ((g >> 1) & 1) ^ 1, 37);
        tc_fence_after_sync();
        if (leader) {
          umma_k128(tmem_base + b * 128, smem_u32(smem + X_OFF), smem_u32(smem + W1_OFF + ws * kOperandTile), idesc, false);
          umma_commit(&w1_empty[ws]);
          umma_commit(&d1_full[b]);
          if (c == 7) umma_commit(x_empty);
        }
        __syncwarp();
      }
    }
  } else if (warp == 18) {
    // ------------------------------------------------------------------ GEMM2 issuer
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      for (int g = 0; g < total_chunks; ++g) {  // consumes H[g&1] and the fc3 slice of chunk g
        const int c = g & 7, b = g & 1, o = (g >> 3) & 1, ws = g % WS;
        mbar_wait(&h_full[b], (g >> 1) & 1, 32);
        mbar_wait(&w3_full[ws], (g / WS) & 1, 33);
        if (c == 0) mbar_wait(&out_empty[o], (((g >> 3) >> 1) & 1) ^ 1, 34);
        tc_fence_after_sync();
        const uint32_t h_s = smem_u32(smem + H_OFF + b * kOperandHalf);
        const uint32_t w3_s = smem_u32(smem + W3_OFF + ws * kOperandHalf);
        const uint32_t h_lo = desc_lo(h_s), w3_lo = desc_lo(w3_s);
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss2(tmem_base + 256 + o * 128, h_lo + 2 * k, kDescHiSw128, w3_lo + 2 * k, kDescHiSw128, idesc, (c | k) != 0);
          umma_commit(&h_empty[b]);
          umma_commit(&w3_empty[ws]);
          if (c == 7) umma_commit(&out_full[o]);
        }
        __syncwarp();
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ producers
    const int pt = threadIdx.x - 256;  // 0..255
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_w, p.ln_b, pt, gamma, beta, 0.5f);
    RowTile<256> regs;
    auto load_tile = [&](int tile) {
      const long long row0 = (long long)tile * 128;
      auto rp = [&](int r) -> const void* {
        return (row0 + r) < p.rows ? static_cast<const uint8_t*>(p.x) + (row0 + r) * kD * zbytes<F32>() : nullptr;
      };
      if (p.use_norm)
        regs.template load<F32, true, 1>(pt, rp, gamma, beta, p.eps);
      else
        regs.template load<F32, false>(pt, rp, gamma, beta, p.eps, 0.5f);
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      mbar_wait(x_empty, (it & 1) ^ 1, 38);
      regs.store_operand(pt, smem + X_OFF);
      fence_proxy_async_smem();
      mbar_arrive(x_full);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    // ------------------------------------------------------------------ SwiGLU epilogues
    // These warps also drain the finished output accumulators: group `grp` owns output channels 64*grp .. +63 and
    // stores them in 64 / CPS parts (CPS columns = 64 B at a time through the group's staging tile and TMA), one
    // part after each of its SwiGLU chunks of the NEXT tile, so the drain of tile i - 1 is spread over tile i
    // and neither the chunk pipeline nor the LayerNorm producers wait for it.
    const int grp = warp >> 2;             // 0: even chunks, 1: odd chunks
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;     // pair row of the tile == TMEM lane
    constexpr int CPS = F32 ? 16 : 32;
    constexpr int PARTS = 64 / CPS;
    const int half = grp;
    const bool leader = (threadIdx.x & 127) == 0;
    const bool reduce = p.add_residual && p.out == p.x;
    const bool read_res = p.add_residual && !reduce;
    const uint32_t row_off = r * 64, row_xor = (r >> 1) & 3;
    uint8_t* stage = smem + STAGE_OFF + half * 8192;
    auto drain_part = [&](int ot, int otile, int k) {  // part k of output tile number `ot` (global tile `otile`)
      const int o = ot & 1;
      const uint32_t o_addr = tmem_addr(tmem_base, quarter * 32, 256 + o * 128 + half * 64);
      if (k == 0) {
        mbar_wait(&out_full[o], (ot >> 1) & 1, 41);
        tc_fence_after_sync();
      }
      const long long row = (long long)otile * 128 + r;
      const bool valid = row < p.rows;
      const uint8_t* xrow = static_cast<const uint8_t*>(p.x) + row * kD * zbytes<F32>();
      uint32_t v[CPS];
      if (F32) tmem_ld_32x16(o_addr + k * CPS, reinterpret_cast<uint32_t(&)[16]>(v));
      else tmem_ld_32x32(o_addr + k * CPS, reinterpret_cast<uint32_t(&)[32]>(v));
      tmem_ld_wait();
      if (k == PARTS - 1) {
        tc_fence_before_sync();
        mbar_arrive(&out_empty[o]);
      }
      const int ch0 = half * 64 + k * CPS;
      float zr[CPS / 8][8];
#pragma unroll
      for (int q = 0; q < CPS / 8; ++q) {
        if (read_res && valid) {
          load8<F32>(xrow, ch0 + q * 8, zr[q]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) zr[q][e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) zr[q][e] = fmaf(2.0f, __uint_as_float(v[q * 8 + e]), zr[q][e]);
      }
      if (leader) tma_store_wait_read0();  // the previous store has read the staging tile
      named_bar_sync(1 + half, 128);
#pragma unroll
      for (int q = 0; q < CPS / 8; ++q) {
        if (F32) {
          *reinterpret_cast<float4*>(stage + row_off + (((q * 2) ^ row_xor) << 4)) =
              make_float4(zr[q][0], zr[q][1], zr[q][2], zr[q][3]);
          *reinterpret_cast<float4*>(stage + row_off + (((q * 2 + 1) ^ row_xor) << 4)) =
              make_float4(zr[q][4], zr[q][5], zr[q][6], zr[q][7]);
        } else {
          *reinterpret_cast<uint4*>(stage + row_off + ((q ^ row_xor) << 4)) =
              make_uint4(pack_bf16x2(zr[q][0], zr[q][1]), pack_bf16x2(zr[q][2], zr[q][3]), pack_bf16x2(zr[q][4], zr[q][5]),
                         pack_bf16x2(zr[q][6], zr[q][7]));
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1 + half, 128);
      if (leader) {
        if (reduce)
          tma_reduce_add_2d(&tmO, stage, ch0, otile * 128);
        else
          tma_store_2d(&tmO, stage, ch0, otile * 128);
        tma_store_commit();
      }
    };
    int it = 0;
    int tile = blockIdx.x;
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      int part = 0;
      for (int c = grp; c < CHUNKS; c += 2) {
        const int g = it * CHUNKS + c;
        const int b = g & 1;  // == grp
        mbar_wait(&d1_full[b], (g >> 1) & 1, 39);
        tc_fence_after_sync();
        mbar_wait(&h_empty[b], ((g >> 1) & 1) ^ 1, 40);
        uint8_t* hrow = smem + H_OFF + b * kOperandHalf;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t av[32], bv[32];
          tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, b * 128 + hh * 32), av);
          tmem_ld_32x32(tmem_addr(tmem_base, quarter * 32, b * 128 + 64 + hh * 32), bv);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j0 = q * 8 + e * 2;
              const float a0 = __uint_as_float(av[j0]), a1 = __uint_as_float(av[j0 + 1]);
              const float u0 = a0 * __uint_as_float(bv[j0]), u1 = a1 * __uint_as_float(bv[j0 + 1]);
              o[e] = pack_bf16x2(fmaf(u0, tanh_approx(a0), u0), fmaf(u1, tanh_approx(a1), u1));
            }
            *reinterpret_cast<uint4*>(hrow + sw128_offset(r, hh * 4 + q)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(&d1_empty[b]);
        mbar_arrive(&h_full[b]);
        // one part of the previous tile's output (4 chunks per group and tile: every part finds its turn)
        if (it > 0 && part < PARTS && (PARTS == 4 || (c >> 1) & 1)) {
          drain_part(it - 1, tile - (int)gridDim.x, part);
          ++part;
        }
      }
    }
    if (it > 0) {  // the last tile's output
#pragma unroll 1
      for (int k = 0; k < PARTS; ++k) drain_part(it - 1, tile - (int)gridDim.x, k);
    }
    if (leader) tma_store_wait0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 16) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200
