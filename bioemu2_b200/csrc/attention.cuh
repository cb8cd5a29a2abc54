// Flash-style attention with an additive pair-bias tile, shared by single-track pair-bias attention
// and triangle attention.
//
//   out[b, q, h, :] = gate * softmax_k( Q[b,q,h,:] . K[b,k,h,:] + bias[b / bias_div, h, q, k] ) V[b,k,h,:]
//
// with keys whose mask byte is zero REPLACED by a finite -1e6 (natural-log units) before the softmax,
// which is what the reference does (a fully masked row averages over all keys, it never produces NaN).
// Q and the bias arrive pre-multiplied by log2(e) (Q also by 1/sqrt(dh)), so the kernel works in base 2.
//
// One work item = (batch b, head h, tile of 128 queries); a persistent CTA walks work items.
//   warps 0-3  softmax: one thread per query row; S tile from TMEM, bias tile from shared memory (TMA,
//              128-byte swizzle), online max/sum in registers, P written as a bf16 MMA operand; the
//              output accumulator lives in registers and takes each key tile's P.V from TMEM
//   warp  4    TMA loader (Q once per item; K, V^T and bias tiles through a ring)
//   warp  5    MMA issuer (S = Q.K^T into one of two TMEM buffers, O_t = P.V into one of two)
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
  int nqt, nkt;
  int total_work;
};

template <int DH>
struct FlashCfg {
  static constexpr int STAGES = (DH == 32) ? 3 : 2;
  static constexpr uint32_t Q_BYTES = 128 * DH * 2;
  static constexpr uint32_t K_BYTES = 128 * DH * 2;
  static constexpr uint32_t V_HALF = DH * 128;           // DH rows x 64 keys x 2 B
  static constexpr uint32_t V_BYTES = 2 * V_HALF;
  static constexpr uint32_t BIAS_BYTES = 2 * kOperandHalf;
  static constexpr uint32_t STAGE_BYTES = K_BYTES + V_BYTES + BIAS_BYTES;
  static constexpr uint32_t Q_OFF = 0;
  static constexpr uint32_t STAGE_OFF = 16384;           // Q region rounded up
  static constexpr uint32_t P_OFF = STAGE_OFF + STAGES * STAGE_BYTES;
  static constexpr uint32_t MASK_OFF = P_OFF + 2 * kOperandTile;  // 2 x 8 words of mask bits
  static constexpr uint32_t BAR_OFF = MASK_OFF + 64;
  static constexpr uint32_t SMEM_BYTES = BAR_OFF + 256 + 1024;
  static constexpr int THREADS = 192;
};

__device__ __forceinline__ uint64_t make_desc_k(uint32_t addr, bool sw64) {
  return sw64 ? make_desc_k_sw64(addr) : make_desc_k_sw128(addr);
}

__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int DH>
__global__ void __launch_bounds__(192, 1)
flash_core_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
                  FlashParams p) {
  using Cfg = FlashCfg<DH>;
  constexpr bool SW64 = (DH == 32);
  constexpr float kNegMasked = -1.0e6f * 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* q_full = bars;            // TMA
  uint64_t* q_empty = bars + 1;       // commit (all S products of the item issued and done)
  uint64_t* kv_full = bars + 2;       // [3] TMA
  uint64_t* kv_empty = bars + 5;      // [3] commit
  uint64_t* s_full = bars + 8;        // [2] commit
  uint64_t* s_empty = bars + 10;      // [2] count 128
  uint64_t* p_full = bars + 12;       // [2] count 128
  uint64_t* p_empty = bars + 14;      // [2] commit
  uint64_t* o_full = bars + 16;       // [2] commit
  uint64_t* o_empty = bars + 18;      // [2] count 128
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  uint32_t* mask_bits = reinterpret_cast<uint32_t*>(smem + Cfg::MASK_OFF);  // [2][4] valid bits, then [2][4] unused

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&p_empty[i], 1);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmBias);
  }
  if (warp == 5) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S[0] 0..127, S[1] 128..255, O_t[0] 256.., O_t[1] 256+DH..

  const int T = p.nkt;
  // Global counters: g counts key tiles over all work items of this CTA (ring slot = g % STAGES,
  // S/P/O buffer = g & 1); w counts work items.

  if (warp == 4) {
    // ------------------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      int g = 0, w = 0;
      for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
        const int qt = work % p.nqt;
        const int bh = work / p.nqt;
        const int h = bh % p.H;
        const int b = bh / p.H;
        mbar_wait(q_empty, (w & 1) ^ 1, 60);
        mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
        tma_load_3d(smem + Cfg::Q_OFF, &tmQ, q_full, p.q_col0 + h * DH, qt * 128, b);
        const int bias_g = (b / p.bias_div) * p.H + h;
        for (int t = 0; t < T; ++t, ++g) {
          const int st = g % Cfg::STAGES;
          mbar_wait(&kv_empty[st], ((g / Cfg::STAGES) & 1) ^ 1, 61);
          uint8_t* base = smem + Cfg::STAGE_OFF + st * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&kv_full[st], Cfg::STAGE_BYTES);
          tma_load_3d(base, &tmK, &kv_full[st], p.k_col0 + h * DH, t * 128, b);
          tma_load_3d(base + Cfg::K_BYTES, &tmV, &kv_full[st], t * 128, p.v_row0 + h * DH, b);
          tma_load_3d(base + Cfg::K_BYTES + Cfg::V_HALF, &tmV, &kv_full[st], t * 128 + 64, p.v_row0 + h * DH, b);
          tma_load_3d(base + Cfg::K_BYTES + Cfg::V_BYTES, &tmBias, &kv_full[st], t * 128, qt * 128, bias_g);
          tma_load_3d(base + Cfg::K_BYTES + Cfg::V_BYTES + kOperandHalf, &tmBias, &kv_full[st], t * 128 + 64,
                      qt * 128, bias_g);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, DH);
      const uint32_t q_s = smem_u32(smem + Cfg::Q_OFF);
      auto issue_s = [&](int g) {  // S[g&1] = Q . K(g)^T
        const int st = g % Cfg::STAGES;
        mbar_wait(&kv_full[st], (g / Cfg::STAGES) & 1, 62);
        mbar_wait(&s_empty[g & 1], ((g >> 1) & 1) ^ 1, 63);
        tc_fence_after_sync();
        const uint32_t k_s = smem_u32(smem + Cfg::STAGE_OFF + st * Cfg::STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16_ss(tmem_base + (g & 1) * 128, make_desc_k(q_s + k * 32, SW64), make_desc_k(k_s + k * 32, SW64),
                       idesc_s, k > 0);
        umma_commit(&s_full[g & 1]);
      };
      int g = 0, w = 0;
      for (int work = blockIdx.x; work < p.total_work; work += gridDim.x, ++w) {
        mbar_wait(q_full, w & 1, 64);
        issue_s(g);
        for (int t = 0; t < T; ++t, ++g) {
          if (t + 1 < T) {
            issue_s(g + 1);
          } else {
            umma_commit(q_empty);  // every S product of this item has been issued
          }
          const int st = g % Cfg::STAGES;
          mbar_wait(&p_full[g & 1], (g >> 1) & 1, 65);
          mbar_wait(&o_empty[g & 1], ((g >> 1) & 1) ^ 1, 66);
          tc_fence_after_sync();
          const uint32_t p_s = smem_u32(smem + Cfg::P_OFF + (g & 1) * kOperandTile);
          const uint32_t v_s = smem_u32(smem + Cfg::STAGE_OFF + st * Cfg::STAGE_BYTES + Cfg::K_BYTES);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_bf16_ss(tmem_base + 256 + (g & 1) * DH,
                         make_desc_k_sw128(p_s + (k >> 2) * kOperandHalf + (k & 3) * 32),
                         make_desc_k_sw128(v_s + (k >> 2) * Cfg::V_HALF + (k & 3) * 32), idesc_o, k > 0);
          umma_commit(&o_full[g & 1]);
          umma_commit(&p_empty[g & 1]);
          umma_commit(&kv_empty[st]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------------------ softmax
    const int r = warp * 32 + lane;  // query row of the tile == TMEM lane
    int g = 0;
    for (int work = blockIdx.x; work < p.total_work; work += gridDim.x) {
      const int qt = work % p.nqt;
      const int bh = work / p.nqt;
      const int h = bh % p.H;
      const int b = bh / p.H;
      const uint8_t* mrow = p.mask + (long long)(b / p.mask_div) * p.mask_row_stride;
      float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
      float o[DH];
#pragma unroll
      for (int d = 0; d < DH; ++d) o[d] = 0.f;

      for (int t = 0; t < T; ++t, ++g) {
        const int buf = g & 1;
        const int st = g % Cfg::STAGES;
        // key-validity bits of this tile: bit j of word w <=> key t*128 + 32*w + j exists and is unmasked
        {
          const int key = t * 128 + r;
          const bool ok = key < p.N && mrow[key * p.mask_key_stride] != 0;
          const bool in = key < p.N;
          const uint32_t okb = __ballot_sync(0xffffffffu, ok);
          const uint32_t inb = __ballot_sync(0xffffffffu, in);
          if (lane == 0) {
            mask_bits[buf * 8 + warp] = okb;
            mask_bits[buf * 8 + 4 + warp] = inb;
          }
        }
        softmax_bar_sync();
        uint32_t okbits[4], inbits[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          okbits[i] = mask_bits[buf * 8 + i];
          inbits[i] = mask_bits[buf * 8 + 4 + i];
        }

        mbar_wait(&s_full[buf], (g >> 1) & 1, 67);
        tc_fence_after_sync();
        float x[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, buf * 128 + c * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) x[c * 32 + j] = __uint_as_float(v[j]);
        }
        tc_fence_before_sync();
        mbar_arrive(&s_empty[buf]);

        mbar_wait(&kv_full[st], (g / Cfg::STAGES) & 1, 68);
        const uint8_t* bias_s = smem + Cfg::STAGE_OFF + st * Cfg::STAGE_BYTES + Cfg::K_BYTES + Cfg::V_BYTES;
        float mx = m_run;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const uint4 bv = *reinterpret_cast<const uint4*>(bias_s + (c >> 3) * kOperandHalf + sw128_offset(r, c & 7));
          const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = c * 8 + e;
            const float bias = (e & 1) ? bf16hi(bw[e >> 1]) : bf16lo(bw[e >> 1]);
            float val = x[j] + bias;
            val = ((okbits[j >> 5] >> (j & 31)) & 1u) ? val : kNegMasked;
            val = ((inbits[j >> 5] >> (j & 31)) & 1u) ? val : -INFINITY;
            x[j] = val;
            mx = fmaxf(mx, val);
          }
        }
        const float alpha = exp2_approx(m_run - mx);
        m_run = mx;
        float sum = 0.f;
        mbar_wait(&p_empty[buf], ((g >> 1) & 1) ^ 1, 69);
        uint8_t* p_s = smem + Cfg::P_OFF + buf * kOperandTile;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float e8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            e8[e] = exp2_approx(x[c * 8 + e] - mx);
            sum += e8[e];
          }
          *reinterpret_cast<uint4*>(p_s + (c >> 3) * kOperandHalf + sw128_offset(r, c & 7)) =
              make_uint4(pack_bf16x2(e8[0], e8[1]), pack_bf16x2(e8[2], e8[3]), pack_bf16x2(e8[4], e8[5]),
                         pack_bf16x2(e8[6], e8[7]));
        }
        l_run = l_run * alpha + sum;
        fence_proxy_async_smem();
        mbar_arrive(&p_full[buf]);

        if (t > 0) {  // fold in the previous key tile's P.V (it was computed relative to the previous max)
          const int pb = (g - 1) & 1;
          mbar_wait(&o_full[pb], ((g - 1) >> 1) & 1, 70);
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, 256 + pb * DH + c * 32), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[c * 32 + j] = fmaf(o[c * 32 + j], alpha_prev, __uint_as_float(v[j]));
          }
          tc_fence_before_sync();
          mbar_arrive(&o_empty[pb]);
        }
        alpha_prev = alpha;
      }
      {  // last key tile's P.V
        const int pb = (g - 1) & 1;
        mbar_wait(&o_full[pb], ((g - 1) >> 1) & 1, 71);
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_addr(tmem_base, warp * 32, 256 + pb * DH + c * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[c * 32 + j] = fmaf(o[c * 32 + j], alpha_prev, __uint_as_float(v[j]));
        }
        tc_fence_before_sync();
        mbar_arrive(&o_empty[pb]);
      }
      const int q = qt * 128 + r;
      if (q < p.N) {
        const float inv_l = 1.0f / l_run;
        __nv_bfloat16* dst = p.out + (long long)b * p.out_b_stride + (long long)q * p.out_pitch + p.out_col0 + h * p.dh_out;
        const __nv_bfloat16* gsrc =
            p.gate ? p.gate + (long long)b * p.gate_b_stride + (long long)q * p.gate_pitch + p.gate_col0 + h * p.dh_out
                   : nullptr;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          if (c * 8 < p.dh_out) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = o[c * 8 + e] * inv_l;
            if (gsrc) {
              const uint4 gv = *reinterpret_cast<const uint4*>(gsrc + c * 8);
              const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
              for (int e = 0; e < 8; ++e)
                y[e] *= sigmoid_fast((e & 1) ? bf16hi(gw[e >> 1]) : bf16lo(gw[e >> 1]));
            }
            *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                                pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// -------------------------------------------------------------------------------------------------
// Pair bias: zb[h][i][j] = scale * proj_z(LN_z(z[i, j, :]))[h] for up to 16 heads, bf16, row pitch Nk.
// A tile is 128 consecutive j of one row i: producers LayerNorm the rows into an MMA operand, one
// 128 x 16 x 128 product per tile, lanes = pairs so every head's row is stored coalesced.
//   warps 0-3 epilogue, warps 4-11 producers, warp 12 control.
struct PairBiasParams {
  const void* z;        // [N][N][128] fp32 or bf16
  const float* ln_w;
  const float* ln_b;    // nullptr: LayerNorm without bias
  __nv_bfloat16* zb;    // [H][N][Nk]
  int N, Nk, H;
  int transposed;       // 1: bias of the transposed pair tensor, zb[h][i][j] from z[j][i]
  int num_tiles;        // N * ceil(N/128)
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
  const int tiles_per_row = (p.N + 127) >> 7;

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
    if (lane == 0) {
      mbar_arrive_expect_tx(w_full, 4096);
      tma_load_2d(smem + W_OFF, &tmW, w_full, 0, 0);
      tma_load_2d(smem + W_OFF + 2048, &tmW, w_full, 64, 0);
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
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + s * 16, make_desc_k_sw128(x_s + (k >> 2) * kOperandHalf + (k & 3) * 32),
                       make_desc_k_sw128(w_s + (k >> 2) * 2048 + (k & 3) * 32), idesc, k > 0);
        umma_commit(&x_empty[s]);
        umma_commit(&acc_full[s]);
      }
    }
  } else if (warp >= 4) {
    const int pt = threadIdx.x - 128;
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_w, p.ln_b, pt, gamma, beta);
    RowTile<256> regs;
    const long long pos_stride = (p.transposed ? (long long)p.N * kD : kD) * (long long)zbytes<F32>();
    const long long line_stride = (p.transposed ? kD : (long long)p.N * kD) * (long long)zbytes<F32>();
    auto load_tile = [&](int tile) {
      const int i = tile / tiles_per_row;
      const int j0 = (tile - i * tiles_per_row) << 7;
      const uint8_t* base = static_cast<const uint8_t*>(p.z) + i * line_stride;
      regs.template load<F32, true>(
          pt, [&](int r) -> const void* { return (j0 + r) < p.N ? base + (j0 + r) * pos_stride : nullptr; },
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
      if (j < p.N) {
#pragma unroll
        for (int h = 0; h < 16; ++h)
          if (h < p.H) p.zb[((long long)h * p.N + i) * p.Nk + j] = __float2bfloat16(__uint_as_float(v[h]) * p.scale);
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
