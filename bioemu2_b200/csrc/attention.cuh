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
// G "softmax groups" of eight warps each own one query tile and share the K / V^T tiles of the item:
//   softmax warps  two threads per query row (one per 64-column half of a score tile), so a thread holds its
//                  whole share of a score tile in registers: one TMEM read per key tile, online max/sum (row
//                  maximum exchanged through shared memory once per key tile), P written back to TMEM as
//                  packed bf16; the output accumulator lives in registers (half the head dim per thread) and
//                  takes each key tile's P.V from TMEM.  Two groups put four softmax warps on every scheduler.
//   loader warp    TMA: Q tiles once per item (two slots, so the next item's arrive early), K and V^T through a
//                  ring, one bias tile per group
//   MMA warp       S_g = Q_g.K^T + bias tile into one of the group's two TMEM score buffers (the bias is added by
//                  the tensor core: eight 128 x 16 x 16 products of the bias tile's 16-column blocks, as the A
//                  operand, with a 16 x 16 identity, each onto its own 16 accumulator columns, so the softmax
//                  threads never touch the bias); O_g = P_g.V with P read from TMEM, where the softmax threads leave it
//                  (packed bf16, in the first 64 columns of the score buffer it was computed from), alternating per key tile, so
//                  the next scores are ready when a softmax pass ends; P_g.V lands in the first DH columns of
//                  the score buffer its P came from (dead by then).  The tile stream runs on across work
//                  items: the first scores of the next item are issued during the last tile of this one.
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
  const __nv_bfloat16* gate;  // raw gate logits (sigmoid applied here) or nullptr
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
  static constexpr int STAGES = (DH == 32) ? 3 : 2;
  static constexpr int MAX_T = 64;                       // key tiles per row: N <= 8192
  static constexpr uint32_t Q_BYTES = 128 * DH * 2;      // per group
  static constexpr uint32_t K_BYTES = 128 * DH * 2;
  static constexpr uint32_t V_HALF = DH * 128;           // DH rows x 64 keys x 2 B
  static constexpr uint32_t V_BYTES = 2 * V_HALF;
  static constexpr uint32_t KV_BYTES = K_BYTES + V_BYTES;
  static constexpr uint32_t Q_OFF = 0;                   // [2 slots][G] query tiles
  static constexpr uint32_t KV_OFF = 2 * G * Q_BYTES;
  static constexpr uint32_t BIAS_OFF = KV_OFF + STAGES * KV_BYTES;   // [G][2 slots] tiles x 32 KB
  static constexpr uint32_t MASK_OFF = BIAS_OFF + 2 * G * kOperandTile;  // 2 x MAX_T x 8 words
  static constexpr uint32_t XCH_OFF = MASK_OFF + 2 * MAX_T * 32;  // per group 768 floats: row max / row sum exchange
  // 16 x 16 identity (bf16) as an unswizzled K-major operand: two 16-byte K chunks of 16 rows each.
  static constexpr uint32_t IDENT_OFF = XCH_OFF + G * 3072;
  static constexpr uint32_t BAR_OFF = IDENT_OFF + 512;
  static constexpr uint32_t SMEM_BYTES = BAR_OFF + 384 + 1024;
  static constexpr int THREADS = 256 * G + 128;        // G softmax groups of 8 warps + loader / MMA / mask (+1 idle) warps
  static constexpr int SOFTMAX_REGS = 0;  // setmaxnreg targets when three warpgroups share the file
  static constexpr int OTHER_REGS = 40;
};

__device__ __forceinline__ uint64_t make_desc_k(uint32_t addr, bool sw64) {
  return sw64 ? make_desc_k_sw64(addr) : make_desc_k_sw128(addr);
}

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
  uint64_t* q_empty = bars + 2;       // [2] commit
  uint64_t* kv_full = bars + 4;       // [3] TMA
  uint64_t* kv_empty = bars + 7;      // [3] commit
  uint64_t* bias_full = bars + 10;    // [G][2 slots] TMA
  uint64_t* bias_empty = bars + 14;   // [G][2] commit
  uint64_t* s_full = bars + 18;       // [G][2 buffers] commit
  uint64_t* s_empty = bars + 22;      // [G][2] count 256: the P.V result in the buffer has been read
  uint64_t* p_full = bars + 26;       // [G] count 256
  uint64_t* o_full = bars + 28;       // [G][2] commit
  uint64_t* mask_full = bars + 32;    // [2] count 1 (mask warp)
  uint64_t* mask_empty = bars + 34;   // [2] count 256*G
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 36);
  // Key-validity bits of a work item's mask row, two buffers of MAX_T x 8 words:
  //   word t*8 + w      bit j <=> key t*128 + 32*w + j exists and is unmasked
  //   word t*8 + 4 + w  bit j <=> key t*128 + 32*w + j exists
  uint32_t* mask_bits = reinterpret_cast<uint32_t*>(smem + Cfg::MASK_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kLoaderWarp = 8 * G;
  constexpr int kMmaWarp = 8 * G + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&p_full[i], 256);
      mbar_init(&mask_full[i], 1);
      mbar_init(&mask_empty[i], 256 * G);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bias_full[i], 1);
      mbar_init(&bias_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 256);
      mbar_init(&o_full[i], 1);
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
  fence_proxy_async_smem();
  if (warp == kMmaWarp) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: score buffer pb of group g at g*256 + pb*128; its first 64 columns later take P (packed bf16),
  // columns 64 .. 64+DH the P.V product.

  const int T = p.nkt;
  // n counts key tiles over all work items of this CTA: every per-tile barrier completes one phase per n
  // (parity n & 1), the K/V ring uses slot n % STAGES; w counts work items.

  // With two softmax warpgroups the register file is re-split (setmaxnreg at the top of each role's
  // branch): the loader/MMA warpgroup gives registers back and each softmax thread gets enough to keep its
  // 128 scores and the output row in registers.
  if (warp >= kLoaderWarp) {
    if (Cfg::SOFTMAX_REGS > 0) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::OTHER_REGS));
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
          const int st = n % Cfg::STAGES;
          mbar_wait(&kv_empty[st], ((n / Cfg::STAGES) & 1) ^ 1, 61);
          uint8_t* base = smem + Cfg::KV_OFF + st * Cfg::KV_BYTES;
          mbar_arrive_expect_tx(&kv_full[st], Cfg::KV_BYTES);
          tma_load_3d(base, &tmK, &kv_full[st], p.k_col0 + h * DH, t * 128, b);
          tma_load_3d(base + Cfg::K_BYTES, &tmV, &kv_full[st], t * 128, p.v_row0 + h * DH, b);
          tma_load_3d(base + Cfg::K_BYTES + Cfg::V_HALF, &tmV, &kv_full[st], t * 128 + 64, p.v_row0 + h * DH, b);
          for (int g = 0; g < G; ++g) {
            const int bs = g * 2 + (n & 1);
            mbar_wait(&bias_empty[bs], ((n >> 1) & 1) ^ 1, 72);
            uint8_t* bb = smem + Cfg::BIAS_OFF + bs * kOperandTile;
            mbar_arrive_expect_tx(&bias_full[bs], kOperandTile);
            tma_load_3d(bb, &tmBias, &bias_full[bs], t * 128, (qg * G + g) * 128, bias_g);
            tma_load_3d(bb + kOperandHalf, &tmBias, &bias_full[bs], t * 128 + 64, (qg * G + g) * 128, bias_g);
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, DH);
      constexpr uint32_t idesc_b = make_idesc_bf16(128, 16);
      // The groups run half a tile out of phase (group 1 starts late, see the softmax code).  The requests of
      // one group are served together: its next score tile, then its P.V.  (One issuing thread per group was
      // measured slower.)  The operand descriptors are stepped by adding to their low words, which keeps this
      // thread's instruction count per MMA small: it shares its scheduler with four busy softmax warps.
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t z_lo = desc_lo(smem_base + Cfg::IDENT_OFF, 256);
      auto issue_s = [&](int n, int g, int qs) {  // S_g(n) = Q_g . K(n)^T into score buffer n & 1
        const int st = n % Cfg::STAGES;
        const int pb = n & 1;
        mbar_wait(&kv_full[st], (n / Cfg::STAGES) & 1, 62);
        mbar_wait(&s_empty[g * 2 + pb], ((n >> 1) & 1) ^ 1, 63);
        tc_fence_after_sync();
        const uint32_t k_lo = desc_lo(smem_base + Cfg::KV_OFF + st * Cfg::KV_BYTES);
        const uint32_t q_lo = desc_lo(smem_base + Cfg::Q_OFF + (qs * G + g) * Cfg::Q_BYTES);
        constexpr uint32_t qk_hi = SW64 ? kDescHiSw64 : kDescHiSw128;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16_ss2(tmem_base + g * 256 + pb * 128, q_lo + 2 * k, qk_hi, k_lo + 2 * k, qk_hi, idesc_s, k > 0);
        // + bias tile: K step k adds bias[:, 16k .. 16k+15] into the same columns of the accumulator
        mbar_wait(&bias_full[g * 2 + pb], (n >> 1) & 1, 68);
        tc_fence_after_sync();
        const uint32_t b_lo = desc_lo(smem_base + Cfg::BIAS_OFF + (g * 2 + pb) * kOperandTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // 128 x 16 x 16: bias columns 16k.. times the 16 x 16 identity, onto the same columns
          umma_bf16_ss2(tmem_base + g * 256 + pb * 128 + 16 * k, b_lo + (k >> 2) * (kOperandHalf >> 4) + (k & 3) * 2,
                        kDescHiSw128, z_lo, desc_hi_noswizzle(128), idesc_b, true);
        umma_commit(&s_full[g * 2 + pb]);
        umma_commit(&bias_empty[g * 2 + pb]);
      };
      int n = 0, w = 0;
      if ((int)blockIdx.x < p.total_work) {
        mbar_wait(&q_full[0], 0, 64);
        for (int g = 0; g < G; ++g) issue_s(0, g, 0);
        if (T == 1) umma_commit(&q_empty[0]);
      }
      for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
        const bool more = work + (int)gridDim.x < p.total_work;
        for (int t = 0; t < T; ++t, ++n) {
          const int st = n % Cfg::STAGES;
          const uint32_t v_lo = desc_lo(smem_base + Cfg::KV_OFF + st * Cfg::KV_BYTES + Cfg::K_BYTES);
          for (int g = 0; g < G; ++g) {
            // next score tile of this group: of this item, or the first one of the next item
            if (t + 1 < T) {
              issue_s(n + 1, g, w & 1);
              if (t + 2 == T && g == G - 1) umma_commit(&q_empty[w & 1]);  // every S product of this item is issued
            } else if (more) {
              if (g == 0) mbar_wait(&q_full[(w + 1) & 1], ((w + 1) >> 1) & 1, 64);
              issue_s(n + 1, g, (w + 1) & 1);
              if (T == 1 && g == G - 1) umma_commit(&q_empty[(w + 1) & 1]);
            }
            mbar_wait(&p_full[g], n & 1, 65);
            tc_fence_after_sync();
            const uint32_t buf = tmem_base + g * 256 + (n & 1) * 128;
#pragma unroll
            for (int k = 0; k < 8; ++k)  // A = P from TMEM: 16 keys = 8 packed columns per K step
              umma_bf16_ts2(buf + 64, buf + k * 8, v_lo + (k >> 2) * (Cfg::V_HALF >> 4) + (k & 3) * 2, kDescHiSw128, idesc_o,
                            k > 0);
            umma_commit(&o_full[g * 2 + (n & 1)]);
          }
          umma_commit(&kv_empty[st]);
        }
      }
    }
  } else if (warp == kMmaWarp + 1) {
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
  }
  } else {
    if (Cfg::SOFTMAX_REGS > 0)
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::SOFTMAX_REGS > 0 ? Cfg::SOFTMAX_REGS : 240));
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
