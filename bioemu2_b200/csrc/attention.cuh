// Flash-style attention with an additive pair-bias tile, shared by single-track pair-bias attention
// and triangle attention.
//
//   out[b, q, h, :] = gate * softmax_k( Q[b,q,h,:] . K[b,k,h,:] + bias[b / bias_div, h, q, k] ) V[b,k,h,:]
//
// with keys whose mask byte is zero REPLACED by a finite -1e6 (natural-log units) before the softmax,
// which is what the reference does (a fully masked row averages over all keys, it never produces NaN).
// Q and the bias arrive pre-multiplied by log2(e) (Q also by 1/sqrt(dh)), so the kernel works in base 2.
//
// One work item = (batch b, head h, G consecutive tiles of 128 queries); a persistent CTA walks work items.
// G "softmax groups" of eight warps each own one query tile and share the K / V^T tiles of the item.
//
// Tensor memory per group: S (128 fp32 columns, one buffer), P (64 columns of packed bf16, the A operand of P.V)
// and the output accumulator O (DH + 16 fp32 columns), which stays in tensor memory for the whole work item.  V^T
// carries a row of ones below its DH rows, so column DH of O is the row sum of P -- the softmax denominator comes
// out of the same product, from the same rounded P, and costs the softmax threads nothing.
//   softmax warps  two threads per query row (one per 64-column half of a score tile, "side").  Per key tile a
//                  thread reads its 64 scores (bias already added by the tensor core) from S once -- S is then free
//                  for the next tile's product -- applies the key mask, finds the row maximum (exchanged with the
//                  other side through shared memory), and writes P = 2^(score - reference) as packed bf16, two
//                  exponentials per instruction.  The reference maximum is only moved when the new maximum exceeds
//                  it by more than kRescaleThreshold ("lazy rescale"): then, and only then, the thread multiplies
//                  its half of the row of O in tensor memory by the correction factor.  In the steady state the
//                  softmax threads never wait for a P.V product and never touch O until the item ends.
//   loader warp    TMA: Q tiles once per item (two slots), K and V^T through rings of their own (K is needed a tile
//                  earlier than V), one bias tile per group and key tile (two slots per group)
//   MMA warps      one per group: S_g = Q_g.K^T + bias tile as soon as the softmax threads have read the previous S_g (the bias is
//                  added by the tensor core: eight 128 x 16 x 16 products of the bias tile's 16-column blocks, as
//                  the A operand, with a 16 x 16 identity, each onto its own 16 accumulator columns); O_g (+)= P_g.V
//                  (8 instructions, A from tensor memory) as soon as P_g is written.  The tile stream runs on
//                  across work items.
//   mask warp      turns the next item's mask row into bit words.
// Head dim is padded to DH = 32 or 64 by the projections (zero rows/columns), V is supplied transposed
// ([DH][keys]) so both products read K-major operands.
#pragma once
#include "row_tile.cuh"

namespace b200 {

struct FlashParams {
  const uint8_t* mask;  // one byte per key: mask[(b / mask_div) * mask_row_stride + key * mask_key_stride]
  int mask_div;
  long long mask_row_stride, mask_key_stride;
  int bias_div;         // bias group of batch item b is b / bias_div
  const __nv_bfloat16* gate;  // gate or nullptr: raw logits (sigmoid applied here), or sigmoid values when gate_activated
  int gate_activated;
  long long gate_b_stride;
  int gate_pitch, gate_col0;
  __nv_bfloat16* out;
  long long out_b_stride;
  int out_pitch, out_col0;
  int dh_out;           // columns actually stored per head (<= DH, multiple of 8)
  int N, H, Bt;
  int q_col0, k_col0, v_row0;
  int nqt, nkt;         // query tiles, key tiles (nkt <= FlashCfg::MAX_T)
  int nqg;              // query-tile groups per (b, h): ceil(nqt / G)
  int total_work;
};

template <int DH, int G>
struct FlashCfg {
  static constexpr int K_STAGES = 3, V_STAGES = 2;
  static constexpr int MAX_T = 64;                       // key tiles per row: N <= 8192
  static constexpr int NV = DH + 16;                     // rows of the V^T operand: DH value rows, one row of ones, 15 of zeros
  static constexpr uint32_t Q_BYTES = 128 * DH * 2;      // per group
  static constexpr uint32_t K_BYTES = 128 * DH * 2;
  static constexpr uint32_t V_HALF = NV * 128;           // NV rows x 64 keys x 2 B
  static constexpr uint32_t V_BYTES = 2 * V_HALF;
  static constexpr uint32_t V_TMA_BYTES = 2 * DH * 128;  // what TMA writes per stage (the value rows of both halves)
  static constexpr uint32_t Q_OFF = 0;                   // [2 slots][G] query tiles
  static constexpr uint32_t K_OFF = 2 * G * Q_BYTES;
  static constexpr uint32_t V_OFF = K_OFF + K_STAGES * K_BYTES;
  static constexpr uint32_t BIAS_OFF = V_OFF + V_STAGES * V_BYTES;   // [G][2 slots] tiles x 32 KB
  static constexpr uint32_t MASK_OFF = BIAS_OFF + 2 * G * kOperandTile;  // 2 x MAX_T x 8 words
  static constexpr uint32_t XCH_OFF = MASK_OFF + 2 * MAX_T * 32;  // per group [tile parity][side][128] floats: row max exchange
  // 16 x 16 identity (bf16) as an unswizzled K-major operand: two 16-byte K chunks of 16 rows each.
  static constexpr uint32_t IDENT_OFF = XCH_OFF + G * 2048;
  static constexpr uint32_t BAR_OFF = IDENT_OFF + 512;
  static constexpr uint32_t SMEM_BYTES = BAR_OFF + 384 + 1024;
  static constexpr int THREADS = 256 * G + 128;        // G softmax groups of 8 warps + loader, MMA (one per group), mask warps
  // tensor-memory columns of one group
  static constexpr uint32_t TM_GROUP = 256;            // column stride between groups (G == 2 needs NV <= 64)
  static constexpr uint32_t TM_S = 0, TM_P = 128, TM_O = 192;   // O: DH value columns, then the row sum
  static_assert(G == 1 || TM_O + NV <= TM_GROUP, "two groups do not fit the tensor memory");
  static_assert(TM_O + NV <= 512, "tensor memory");
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};

// A new maximum becomes the reference only when it exceeds the old one by more than this (base-2 logits): P then
// stays below 2^threshold relative to the reference, O is rescaled rarely, and the exponents that matter keep a fine
// bf16 grid (|score - reference| < 2 has a spacing of 2^-7 or better).
constexpr float kRescaleThreshold = 1.0f;

__device__ __forceinline__ float max8(const float* v, float m) {
  return max3(max3(v[0], v[1], v[2]), max3(v[3], v[4], v[5]), max3(v[6], v[7], m));
}

template <int DH, int G>
__global__ void __launch_bounds__(256 * G + 128, 1)
flash_core_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
                  FlashParams p) {
  using Cfg = FlashCfg<DH, G>;
  constexpr bool SW64 = (DH == 32);
  constexpr float kNegMasked = -1.0e6f * 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* q_full = bars;            // [2 slots] TMA (all G query tiles)
  uint64_t* q_empty = bars + 2;       // [2] one commit per group
  uint64_t* k_full = bars + 4;        // [3] TMA
  uint64_t* k_empty = bars + 7;       // [3] one commit per group: its Q.K^T of the tile has completed
  uint64_t* v_full = bars + 10;       // [2] TMA
  uint64_t* v_empty = bars + 12;      // [2] one commit per group: its P.V of the tile has completed
  uint64_t* bias_full = bars + 14;    // [G][2 slots] TMA
  uint64_t* bias_empty = bars + 18;   // [G][2] commit
  uint64_t* s_full = bars + 22;       // [G] commit: S_g of the current key tile (bias included) is in tensor memory
  uint64_t* s_empty = bars + 24;      // [G] count 256: every softmax thread of the group has read its scores
  uint64_t* p_full = bars + 26;       // [G] count 256: P_g is written (and O_g rescaled if it had to be)
  uint64_t* pv_done = bars + 28;      // [G] commit: O_g += P_g.V of the current key tile has completed
  uint64_t* mask_full = bars + 30;    // [2] count 1 (mask warp)
  uint64_t* mask_empty = bars + 32;   // [2] count 256*G
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 34);
  // Key-validity bits of a work item's mask row, two buffers of MAX_T x 8 words:
  //   word t*8 + w      bit j <=> key t*128 + 32*w + j exists and is unmasked
  //   word t*8 + 4 + w  bit j <=> key t*128 + 32*w + j exists
  uint32_t* mask_bits = reinterpret_cast<uint32_t*>(smem + Cfg::MASK_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kLoaderWarp = 8 * G;
  constexpr int kMmaWarp = 8 * G + 1;     // issues for group 0; group 1 (if any) has its own issuing warp, 8 * G + 3
  constexpr int kMaskWarp = 8 * G + 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], G);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], G);
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], G);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 256);
      mbar_init(&p_full[i], 256);
      mbar_init(&pv_done[i], 1);
      mbar_init(&mask_full[i], 1);
      mbar_init(&mask_empty[i], 256 * G);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bias_full[i], 1);
      mbar_init(&bias_empty[i], 1);
    }
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmBias);
  }
  if (threadIdx.x < 32) {  // identity: 16-byte unit u = (K chunk c, row i) holds K indices 8c .. 8c+7 of row i
    const int c = threadIdx.x >> 4, i = threadIdx.x & 15;
    uint32_t wds[4] = {0, 0, 0, 0};
    if ((i >> 3) == c) wds[(i & 7) >> 1] = (i & 1) ? 0x3F800000u : 0x00003F80u;
    *reinterpret_cast<uint4*>(smem + Cfg::IDENT_OFF + c * 256 + i * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
  }
  // Below the DH value rows of every V^T half tile: a row of ones (bf16 1.0) and 15 rows of zeros, written once --
  // TMA only ever writes the value rows.  16 rows x 128 B = 128 16-byte units per half tile.
  for (int u = threadIdx.x; u < Cfg::V_STAGES * 2 * 128; u += blockDim.x) {
    const int half = u >> 7, unit = u & 127;
    const uint32_t one2 = unit < 8 ? 0x3F803F80u : 0u;  // units 0..7 are row 0 of the block
    *reinterpret_cast<uint4*>(smem + Cfg::V_OFF + half * Cfg::V_HALF + DH * 128 + unit * 16) = make_uint4(one2, one2, one2, one2);
  }
  fence_proxy_async_smem();
  if (warp == kMmaWarp) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int T = p.nkt;
  // n counts key tiles over all work items of this CTA: every per-tile barrier completes one phase per n
  // (parity n & 1), the K/V ring uses slot n % STAGES, the bias slots alternate with n; w counts work items.

  if (warp == kLoaderWarp) {
    // ------------------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      int n = 0, w = 0;
      for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
        const int qg = work % p.nqg;
        const int bh = work / p.nqg;
        const int h = bh % p.H;
        const int b = bh / p.H;
        const int qs = w & 1;
        mbar_wait(&q_empty[qs], ((w >> 1) & 1) ^ 1, 60);
        mbar_arrive_expect_tx(&q_full[qs], G * Cfg::Q_BYTES);
        for (int g = 0; g < G; ++g)
          tma_load_3d(smem + Cfg::Q_OFF + (qs * G + g) * Cfg::Q_BYTES, &tmQ, &q_full[qs], p.q_col0 + h * DH,
                      (qg * G + g) * 128, b);
        const int bias_g = (b / p.bias_div) * p.H + h;
        for (int t = 0; t < T; ++t, ++n) {
          const int ks = n % Cfg::K_STAGES, vs = n % Cfg::V_STAGES;
          mbar_wait(&k_empty[ks], ((n / Cfg::K_STAGES) & 1) ^ 1, 61);
          mbar_arrive_expect_tx(&k_full[ks], Cfg::K_BYTES);
          tma_load_3d(smem + Cfg::K_OFF + ks * Cfg::K_BYTES, &tmK, &k_full[ks], p.k_col0 + h * DH, t * 128, b);
          for (int g = 0; g < G; ++g) {
            const int bs = g * 2 + (n & 1);
            mbar_wait(&bias_empty[bs], ((n >> 1) & 1) ^ 1, 72);
            uint8_t* bb = smem + Cfg::BIAS_OFF + bs * kOperandTile;
            mbar_arrive_expect_tx(&bias_full[bs], kOperandTile);
            tma_load_3d(bb, &tmBias, &bias_full[bs], t * 128, (qg * G + g) * 128, bias_g);
            tma_load_3d(bb + kOperandHalf, &tmBias, &bias_full[bs], t * 128 + 64, (qg * G + g) * 128, bias_g);
          }
          mbar_wait(&v_empty[vs], ((n / Cfg::V_STAGES) & 1) ^ 1, 75);
          uint8_t* vb = smem + Cfg::V_OFF + vs * Cfg::V_BYTES;
          mbar_arrive_expect_tx(&v_full[vs], Cfg::V_TMA_BYTES);
          tma_load_3d(vb, &tmV, &v_full[vs], t * 128, p.v_row0 + h * DH, b);
          tma_load_3d(vb + Cfg::V_HALF, &tmV, &v_full[vs], t * 128 + 64, p.v_row0 + h * DH, b);
        }
      }
    }
  } else if (warp == kMmaWarp || (G == 2 && warp == kMmaWarp + 2)) {
    // ------------------------------------------------------------------------------ MMA issuers, one warp per group
    // The whole warp walks the group's tile stream and waits on the barriers; one elected lane issues the products
    // and the commits.  Keeping the warp converged keeps addresses and descriptors warp-uniform, which keeps the
    // instruction count per MMA small: the warp shares its scheduler with four busy softmax warps.  A warp per
    // group keeps a stall of one group (its threads are busy with an item's epilogue) from holding up the other.
    {
      const int g = (warp == kMmaWarp) ? 0 : 1;
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, Cfg::NV);
      constexpr uint32_t idesc_b = make_idesc_bf16(128, 16);
      constexpr uint32_t qk_hi = SW64 ? kDescHiSw64 : kDescHiSw128;
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t z_lo = desc_lo(smem_base + Cfg::IDENT_OFF, 256);
      const uint32_t tg = tmem_base + g * Cfg::TM_GROUP;
      auto issue_s = [&](int n, int qs) {  // S_g(n) = Q_g . K(n)^T + bias tile
        const int ks = n % Cfg::K_STAGES;
        const int bs = g * 2 + (n & 1);
        const uint32_t k_lo = desc_lo(smem_base + Cfg::K_OFF + ks * Cfg::K_BYTES);
        const uint32_t q_lo = desc_lo(smem_base + Cfg::Q_OFF + (qs * G + g) * Cfg::Q_BYTES);
        const uint32_t b_lo = desc_lo(smem_base + Cfg::BIAS_OFF + bs * kOperandTile);
        mbar_wait(&k_full[ks], (n / Cfg::K_STAGES) & 1, 62);
        mbar_wait(&s_empty[g], (n & 1) ^ 1, 63);   // the scores of tile n - 1 have been read
        mbar_wait(&bias_full[bs], (n >> 1) & 1, 68);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int k = 0; k < DH / 16; ++k)
            umma_bf16_ss2(tg + Cfg::TM_S, q_lo + 2 * k, qk_hi, k_lo + 2 * k, qk_hi, idesc_s, k > 0);
          umma_commit(&k_empty[ks]);
          // + bias tile: step k adds bias[:, 16k .. 16k+15] onto the same columns of the accumulator
#pragma unroll
          for (int k = 0; k < 8; ++k)  // 128 x 16 x 16: bias columns 16k.. times the 16 x 16 identity
            umma_bf16_ss2(tg + Cfg::TM_S + 16 * k, b_lo + (k >> 2) * (kOperandHalf >> 4) + (k & 3) * 2, kDescHiSw128, z_lo,
                          desc_hi_noswizzle(128), idesc_b, true);
          umma_commit(&s_full[g]);
          umma_commit(&bias_empty[bs]);
        }
        __syncwarp();
      };
      int n = 0, w = 0;
      if ((int)blockIdx.x < p.total_work) {
        mbar_wait(&q_full[0], 0, 64);
        issue_s(0, 0);
        if (T == 1 && leader) umma_commit(&q_empty[0]);
      }
      for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
        const bool more = work + (int)gridDim.x < p.total_work;
        for (int t = 0; t < T; ++t, ++n) {
          const int vs = n % Cfg::V_STAGES;
          const uint32_t v_lo = desc_lo(smem_base + Cfg::V_OFF + vs * Cfg::V_BYTES);
          // next score tile of the group: of this item, or the first one of the next item
          if (t + 1 < T) {
            issue_s(n + 1, w & 1);
            if (t + 2 == T && leader) umma_commit(&q_empty[w & 1]);  // every S product of this item is issued
          } else if (more) {
            mbar_wait(&q_full[(w + 1) & 1], ((w + 1) >> 1) & 1, 64);
            issue_s(n + 1, (w + 1) & 1);
            if (T == 1 && leader) umma_commit(&q_empty[(w + 1) & 1]);
          }
          mbar_wait(&p_full[g], n & 1, 65);
          mbar_wait(&v_full[vs], (n / Cfg::V_STAGES) & 1, 66);
          tc_fence_after_sync();
          if (leader) {
#pragma unroll
            for (int k = 0; k < 8; ++k)  // A = P from tensor memory: 16 keys = 8 packed columns per K step
              umma_bf16_ts2(tg + Cfg::TM_O, tg + Cfg::TM_P + k * 8, v_lo + (k >> 2) * (Cfg::V_HALF >> 4) + (k & 3) * 2,
                            kDescHiSw128, idesc_o, (t | k) != 0);  // the item's first product overwrites O
            umma_commit(&pv_done[g]);
            umma_commit(&v_empty[vs]);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == kMaskWarp) {
    // ------------------------------------------------------------------------------ mask warp
    // Turns the next work item's mask row into bit words while the softmax groups work on the current one.
    int w = 0;
    for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
      const int b = (work / p.nqg) / p.H;
      const uint8_t* mrow = p.mask + (long long)(b / p.mask_div) * p.mask_row_stride;
      uint32_t* mb = mask_bits + (w & 1) * Cfg::MAX_T * 8;
      mbar_wait(&mask_empty[w & 1], ((w >> 1) & 1) ^ 1, 74);
      for (int t = 0; t < T; ++t) {
        uint8_t mv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int key = t * 128 + u * 32 + lane;
          mv[u] = key < p.N ? mrow[key * p.mask_key_stride] : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bool in = (t * 128 + u * 32 + lane) < p.N;
          const uint32_t okb = __ballot_sync(0xffffffffu, in && mv[u] != 0);
          const uint32_t inb = __ballot_sync(0xffffffffu, in);
          if (lane == 0) {
            mb[t * 8 + u] = okb;
            mb[t * 8 + 4 + u] = inb;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&mask_full[w & 1]);
    }
  } else if (warp < kLoaderWarp) {
#include "attention_softmax.inc"
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200
