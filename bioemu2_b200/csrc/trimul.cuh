// Triangle multiplication, the two kernels either side of the per-channel
// contraction (which is bmm_nt_kernel):
//
//   trimul_in_kernel   h = LN_in(z);  ab = mask * p_in(h) * sigmoid(g_in(h))
//                      written channel-major, a[d][line][pos] / b[d][line][pos] (bf16, pitch Np),
//                      so that the contraction reads K-major rows.  The product is computed
//                      transposed -- weights are the M operand, the pair tile the N operand -- so
//                      a TMEM lane is an output channel and each thread stores contiguous pairs.
//   trimul_out_kernel  out = p_out(LN_out(t)) * sigmoid(g_out(LN_in(z))) [+ z]
//                      reading t channel-major and writing the pair-major result.
//
// "line/pos": outgoing contracts the column index, a[d][i][k] = ab[i,k,d]; incoming contracts the
// row index, a[d][i][k] = ab[k,i,d].  A tile is 128 consecutive `pos` on one `line`.
#pragma once
#include "row_tile.cuh"

namespace b200 {

// Geometry is given as lines x positions over a (possibly rectangular, possibly strided) slab of the pair
// tensor: pair (line, pos) sits at z + line*z_line_stride + pos*z_pos_stride (bytes), its mask byte at
// mask + line*m_line_stride + pos*m_pos_stride.  Outgoing: line = row, pos = column; incoming: line =
// column, pos = row.
struct TriMulInParams {
  const void* z;           // z stream (fp32 or bf16), 128 channels per pair
  const uint8_t* mask;     // non-zero = valid
  const float* ln_w;
  const float* ln_b;
  __nv_bfloat16* a_out;    // [128][lines_alloc][pos_pitch]
  __nv_bfloat16* b_out;
  int n_lines, n_pos;
  int lines_alloc, pos_pitch;  // pos_pitch: multiple of 128 >= n_pos
  long long z_line_stride, z_pos_stride;
  long long m_line_stride, m_pos_stride;
  int num_tiles;           // n_lines * pos_pitch/128
  float eps;
};

namespace trimul_in {
constexpr uint32_t W_OFF = 0;                       // 4 M-tiles x 32 KB
constexpr uint32_t X_OFF = 4 * kOperandTile;        // 2 stages x 32 KB
constexpr uint32_t MASK_OFF = X_OFF + 2 * kOperandTile;  // 4 stages x 128 B
constexpr uint32_t BAR_OFF = MASK_OFF + 4 * 128;
constexpr uint32_t FLAG_OFF = BAR_OFF + 96;          // 4 stages x 4 "every pair of this quarter valid" bytes
constexpr uint32_t STAGE_OFF = MASK_OFF + 1024;      // per epilogue group a 16 KB tile [128 channels][64 pairs]
constexpr uint32_t SMEM_BYTES = STAGE_OFF + 2 * kOperandHalf + 1024;
constexpr int THREADS = 512;  // warps 0-3 epilogue of a, 4-7 epilogue of b (their first threads issue the MMAs), 8-15 producers
}  // namespace trimul_in

// The LayerNorm output is halved (exactly) before the projections, so the accumulators hold p/2 and g/2
// and the gate is p * sigmoid(g) = p/2 + p/2 * tanh(g/2): one MUFU and one FMA per element.
// 512 threads, not 544: a 17th warp would round the register allocation up to 640 threads and cap every
// thread at 96 registers, which the LayerNorm producers spill at.  So there is no control warp: the first
// thread of each epilogue group issues the two products of its own half (whose accumulators it has just
// drained), and shared stage x is released when both have committed.
template <bool F32>
__global__ void __launch_bounds__(512, 1)
trimul_in_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                 const __grid_constant__ CUtensorMap tmB, TriMulInParams p) {
  using namespace trimul_in;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* x_full = w_full + 1;     // [2]
  uint64_t* x_empty = x_full + 2;    // [2]
  uint64_t* acc_full = x_empty + 2;  // [2]  a-half, b-half
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint8_t* mask_s = smem + MASK_OFF;
  uint8_t* flag_s = smem + FLAG_OFF;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_line = p.pos_pitch >> 7;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&x_full[i], 256);
      mbar_init(&x_empty[i], 2);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    fence_mbar_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    // ------------------------------------------------------------------ producers
    const int pt = threadIdx.x - 256;  // 0..255
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_w, p.ln_b, pt, gamma, beta, 0.5f);
    const long long pos_stride = p.z_pos_stride, line_stride = p.z_line_stride;
    const long long mpos_stride = p.m_pos_stride, mline_stride = p.m_line_stride;
    RowTile<256> regs;
    uint8_t mreg = 0;
    auto load_tile = [&](int tile) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      const uint8_t* base = static_cast<const uint8_t*>(p.z) + line * line_stride;
      regs.template load<F32, true, 8>(
          pt,
          [&](int r) -> const void* {
            const int pos = pos0 + r;
            return pos < p.n_pos ? base + pos * pos_stride : nullptr;
          },
          gamma, beta, p.eps);
      if (pt < 128) {
        const int pos = pos0 + pt;
        mreg = (pos < p.n_pos) ? p.mask[line * mline_stride + pos * mpos_stride] : 0;
      }
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&x_empty[s], ((it >> 1) & 1) ^ 1, 13);
      regs.store_operand(pt, smem + X_OFF + s * kOperandTile);
      if (pt < 128) {
        mask_s[(it & 3) * 128 + pt] = mreg;
        const bool quarter_valid = __all_sync(0xffffffffu, mreg != 0);
        if (lane == 0) flag_s[(it & 3) * 4 + (pt >> 5)] = quarter_valid ? 1 : 0;
      }
      fence_proxy_async_smem();
      mbar_arrive(&x_full[s]);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // Group 0 (warps 0-3) gates and stores the a half, group 1 (warps 4-7) the b half, concurrently.  Lane =
    // channel, columns = pairs; 16 columns at a time with the next chunk's TMEM loads in flight.  The gated
    // values go to the group's swizzled [128 channels][64 pairs] staging tile and leave by TMA store (a row
    // per channel of the channel-major plane).
    const int half = warp >> 2;
    const int d = (warp & 3) * 32 + lane;  // channel inside the half == TMEM lane
    uint8_t* stage = smem + STAGE_OFF + half * kOperandHalf;
    const CUtensorMap* tmOut = half ? &tmB : &tmA;
    const uint32_t p_addr = tmem_addr(tmem_base, (warp & 3) * 32, (half * 2) * 128);
    const uint32_t g_addr = p_addr + 128;
    // The first WARP of the group issues the group's products: all its lanes wait on the barriers and one elected
    // lane issues (a converged warp issues a tcgen05.mma several times faster than a lone thread of a diverged one).
    const bool issue_warp = (warp & 3) == 0;
    const bool leader = issue_warp && elect_one();
    constexpr uint32_t idesc = make_idesc_bf16(128, 128);
    const uint32_t w_s = smem_u32(smem + W_OFF);
    if (issue_warp) {
      if (half == 0 && leader) {
        mbar_arrive_expect_tx(w_full, 4 * kOperandTile);
        for (int mt = 0; mt < 4; ++mt)
          for (int h = 0; h < 2; ++h)
            tma_load_2d(smem + W_OFF + mt * kOperandTile + h * kOperandHalf, &tmW, w_full, h * 64, mt * 128);
      }
      __syncwarp();
      mbar_wait(w_full, 0, 10);
    }
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      const uint32_t* msk = reinterpret_cast<const uint32_t*>(mask_s + (it & 3) * 128);
      if (issue_warp) {  // this half's products for the tile: p and g projections against operand stage it & 1
        const int s = it & 1;
        mbar_wait(&x_full[s], (it >> 1) & 1, 11);
        mbar_wait(&acc_empty[half], (it & 1) ^ 1, 12);  // the whole group has drained the previous tile
        tc_fence_after_sync();
        const uint32_t x_s = smem_u32(smem + X_OFF + s * kOperandTile);
        if (leader) {
          umma_k128(tmem_base + (half * 2) * 128, w_s + (half * 2) * kOperandTile, x_s, idesc, false);
          umma_k128(tmem_base + (half * 2 + 1) * 128, w_s + (half * 2 + 1) * kOperandTile, x_s, idesc, false);
          umma_commit(&acc_full[half]);
          umma_commit(&x_empty[s]);
        }
      }
      __syncwarp();
      mbar_wait(&acc_full[half], it & 1, 14);
      tc_fence_after_sync();
      // every pair of the tile unmasked?  (tiles away from the padding are, and then no select is needed)
      const bool all_valid = *reinterpret_cast<const uint32_t*>(flag_s + (it & 3) * 4) == 0x01010101u;
      uint32_t pa[16], ga[16], pb[16], gb[16];
      tmem_ld_32x16(p_addr, pa);
      tmem_ld_32x16(g_addr, ga);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t(&pv)[16] = (c & 1) ? pb : pa;
        uint32_t(&gv)[16] = (c & 1) ? gb : ga;
        tmem_ld_wait();
        if (c < 7) {
          tmem_ld_32x16(p_addr + (c + 1) * 16, (c & 1) ? pa : pb);
          tmem_ld_32x16(g_addr + (c + 1) * 16, (c & 1) ? ga : gb);
        } else {
          tc_fence_before_sync();
          mbar_arrive(&acc_empty[half]);
        }
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float h0 = __uint_as_float(pv[j]), h1 = __uint_as_float(pv[j + 1]);
          float v0 = fmaf(h0, tanh_approx(__uint_as_float(gv[j])), h0);
          float v1 = fmaf(h1, tanh_approx(__uint_as_float(gv[j + 1])), h1);
          if (!all_valid) {
            const uint32_t m4 = msk[(c * 16 + j) >> 2];
            v0 = ((m4 >> ((j & 3) * 8)) & 0xff) ? v0 : 0.f;
            v1 = ((m4 >> (((j + 1) & 3) * 8)) & 0xff) ? v1 : 0.f;
          }
          packed[j >> 1] = pack_bf16x2(v0, v1);
        }
        if ((c & 3) == 0) {  // the previous store has finished reading the staging tile (its wait hides behind the
          if (d == 0) tma_store_wait_read0();  // chunk's arithmetic above)
          named_bar_sync(1 + half, 128);
        }
        *reinterpret_cast<uint4*>(stage + sw128_offset(d, (c & 3) * 2)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(stage + sw128_offset(d, (c & 3) * 2 + 1)) =
            make_uint4(packed[4], packed[5], packed[6], packed[7]);
        if ((c & 3) == 3) {
          fence_proxy_async_smem();
          named_bar_sync(1 + half, 128);
          if (d == 0) {
            tma_store_3d(tmOut, stage, pos0 + (c >> 2) * 64, line, 0);
            tma_store_commit();
          }
        }
      }
    }
    if (d == 0) tma_store_wait0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------

// Same lines x positions geometry as TriMulInParams; t is [128][lines_alloc][pos_pitch] (tensor map) and is
// indexed by (line, pos), so a transposed t goes with line = column, pos = row.
struct TriMulOutParams {
  const void* z;           // z stream: input of the op (gate and, optionally, residual)
  void* out;               // same dtype and strides as z, may alias it
  const float* ln_in_w;
  const float* ln_in_b;
  const float* ln_out_w;
  const float* ln_out_b;
  int n_lines, n_pos, pos_pitch;
  long long z_line_stride, z_pos_stride;
  int num_tiles;           // n_lines * pos_pitch/128
  int add_residual;
  int pos_is_dim1;         // the output tensor map is {channel, pos, line} (1) or {channel, line, pos} (0)
  float eps;
};

namespace trimul_out {
constexpr uint32_t W_OFF = 0;                          // p_out, g_out: 2 x 32 KB
constexpr uint32_t T_OFF = 2 * kOperandTile;           // raw t tiles [128 d][128 j], 2 stages
constexpr uint32_t A1_OFF = T_OFF + 2 * kOperandTile;  // LN_out(t) operand
constexpr uint32_t A2_OFF = A1_OFF + kOperandTile;     // LN_in(z) operand
constexpr uint32_t LN_OFF = A2_OFF + kOperandTile;     // gamma_out[128], beta_out[128] fp32
constexpr uint32_t BAR_OFF = LN_OFF + 1024;
constexpr uint32_t STAGE_OFF = LN_OFF + 2048;          // 2 x 16 KB output tiles [128 pairs][128 B of channels]
constexpr uint32_t SMEM_BYTES = STAGE_OFF + 2 * kOperandHalf + 1024;
constexpr int THREADS = 512;  // warps 0-3 epilogue (thread 0 also issues the TMA loads and MMAs), 4-7 t transformers, 8-15 z producers
}  // namespace trimul_out

template <bool F32>
__global__ void __launch_bounds__(512, 1)
trimul_out_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmT,
                  const __grid_constant__ CUtensorMap tmO, TriMulOutParams p) {
  using namespace trimul_out;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* t_full = w_full + 1;     // [2] TMA landed a raw t tile
  uint64_t* t_empty = t_full + 2;    // [2] transformers are done with it
  uint64_t* a1_full = t_empty + 2;   // LN_out(t) operand written
  uint64_t* a2_full = a1_full + 1;   // LN_in(z) operand written
  uint64_t* a_empty = a2_full + 1;   // both operands consumed by the MMAs
  uint64_t* acc_full = a_empty + 1;  // [2]
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* ln_s = reinterpret_cast<float*>(smem + LN_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_line = p.pos_pitch >> 7;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], 128);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    mbar_init(a1_full, 128);
    mbar_init(a2_full, 256);
    mbar_init(a_empty, 1);
    fence_mbar_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmT);
    prefetch_tmap(&tmO);
  }
  if (threadIdx.x < 128) {
    ln_s[threadIdx.x] = p.ln_out_w[threadIdx.x];
    ln_s[128 + threadIdx.x] = p.ln_out_b[threadIdx.x];
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ t transformers
    // The raw tile is [d][j] (channel-major, as the contraction writes it); LayerNorm runs over d and the result is row
    // j of A1.  A thread owns TWO adjacent pair columns and HALF of the channels (lanes l and l ^ 16 share a column
    // pair): one 32-bit shared-memory load brings both columns of a channel (two passes of 64 loads where one column
    // per thread took two passes of 128 16-bit loads), and the two half sums meet in one shuffle.
    const int tt = threadIdx.x - 128;
    const int j0 = (tt >> 5) * 32 + (lane & 15) * 2;  // columns j0, j0 + 1
    const int dh = lane >> 4;                         // channels 64*dh .. 64*dh + 63
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int s = it & 1;
      mbar_wait(&t_full[s], (it >> 1) & 1, 25);
      const uint32_t* traw = reinterpret_cast<const uint32_t*>(smem + T_OFF + s * kOperandTile) + (j0 >> 1);
      const uint32_t* tcol = traw + dh * 64 * 64;
      const uint32_t first = traw[0];
      const float shift0 = bf16lo(first), shift1 = bf16hi(first);
      float s0 = 0.f, q0 = 0.f, s1 = 0.f, q1 = 0.f;
#pragma unroll 16
      for (int k = 0; k < 64; ++k) {
        const uint32_t vk = tcol[k * 64];
        const float x0 = bf16lo(vk) - shift0, x1 = bf16hi(vk) - shift1;
        s0 += x0;
        q0 = fmaf(x0, x0, q0);
        s1 += x1;
        q1 = fmaf(x1, x1, q1);
      }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 16);
      q0 += __shfl_xor_sync(0xffffffffu, q0, 16);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
      q1 += __shfl_xor_sync(0xffffffffu, q1, 16);
      const float ms0 = s0 * (1.0f / kD), ms1 = s1 * (1.0f / kD);
      const float rstd0 = rsqrtf(fmaxf(q0 * (1.0f / kD) - ms0 * ms0, 0.f) + p.eps);
      const float rstd1 = rsqrtf(fmaxf(q1 * (1.0f / kD) - ms1 * ms1, 0.f) + p.eps);
      const float mean0 = ms0 + shift0, mean1 = ms1 + shift1;
      mbar_wait(a_empty, (it & 1) ^ 1, 26);
      uint8_t* a1 = smem + A1_OFF + dh * kOperandHalf;  // this thread's channels are one 64-channel half of the operand
#pragma unroll 2
      for (int cc = 0; cc < 8; ++cc) {
        float y0[8], y1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = cc * 8 + i, d = dh * 64 + k;
          const uint32_t vk = tcol[k * 64];
          const float g = ln_s[d], bb = ln_s[128 + d];
          y0[i] = fmaf((bf16lo(vk) - mean0) * rstd0, g, bb);
          y1[i] = fmaf((bf16hi(vk) - mean1) * rstd1, g, bb);
        }
        *reinterpret_cast<uint4*>(a1 + sw128_offset(j0, cc)) = make_uint4(
            pack_bf16x2(y0[0], y0[1]), pack_bf16x2(y0[2], y0[3]), pack_bf16x2(y0[4], y0[5]), pack_bf16x2(y0[6], y0[7]));
        *reinterpret_cast<uint4*>(a1 + sw128_offset(j0 + 1, cc)) = make_uint4(
            pack_bf16x2(y1[0], y1[1]), pack_bf16x2(y1[2], y1[3]), pack_bf16x2(y1[4], y1[5]), pack_bf16x2(y1[6], y1[7]));
      }
      fence_proxy_async_smem();
      mbar_arrive(a1_full);
      mbar_arrive(&t_empty[s]);
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ z producers: LN_in(z) -> A2
    const int pt = threadIdx.x - 256;  // 0..255
    float gamma[8], beta[8];
    load_gamma_beta(p.ln_in_w, p.ln_in_b, pt, gamma, beta);
    RowTile<256> regs;
    auto load_tile = [&](int tile) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      const uint8_t* base = static_cast<const uint8_t*>(p.z) + line * p.z_line_stride + pos0 * p.z_pos_stride;
      regs.template load<F32, true, 8>(
          pt,
          [&](int r) -> const void* { return (pos0 + r) < p.n_pos ? base + r * p.z_pos_stride : nullptr; },
          gamma, beta, p.eps);
    };
    int it = 0;
    int tile = blockIdx.x;
    if (tile < p.num_tiles) load_tile(tile);
    for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
      mbar_wait(a_empty, (it & 1) ^ 1, 27);
      regs.store_operand(pt, smem + A2_OFF);
      fence_proxy_async_smem();
      mbar_arrive(a2_full);
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) load_tile(next);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // Lane = pair, columns = channels.  16 channels at a time with the next chunk's TMEM loads in flight; the
    // gated update goes to a swizzled [128 pairs][128 B] staging tile and leaves by TMA, two tiles in
    // rotation: added into z in place when the residual is wanted and out aliases z (a bulk reduce, so z is
    // not read here), stored otherwise (with the residual added here from global memory if it is wanted).
    constexpr int CPS = F32 ? 2 : 4;  // 16-channel chunks per staging tile (128 B of channels per pair)
    const int r = warp * 32 + lane;   // pair row of the tile == TMEM lane
    const bool reduce = p.add_residual && p.out == p.z;
    const bool read_res = p.add_residual && !reduce;
    // There is no control warp (a 17th warp would cap every thread at 96 registers): thread 0 issues the TMA
    // loads of the weights and the raw t tiles and, in step i, the two products of tile i; the four warps then
    // drain tile i - 1, whose products ran while tile i's operands were being written.
    constexpr uint32_t idesc = make_idesc_bf16(128, 128);
    const uint32_t w_s = smem_u32(smem + W_OFF);
    const uint32_t a1_s = smem_u32(smem + A1_OFF);
    const uint32_t a2_s = smem_u32(smem + A2_OFF);
    auto issue_t = [&](int tile, int s) {
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      mbar_arrive_expect_tx(&t_full[s], kOperandTile);
      tma_load_3d(smem + T_OFF + s * kOperandTile, &tmT, &t_full[s], pos0, line, 0);
    };
    int my_tiles = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) ++my_tiles;
    // Warp 0 as a whole waits on the barriers; one elected lane issues the loads and the products (a converged warp
    // issues a tcgen05.mma several times faster than a lone thread of a diverged one).
    const bool leader = warp == 0 && elect_one();
    if (warp == 0) {
      if (leader) {
        mbar_arrive_expect_tx(w_full, 2 * kOperandTile);
        for (int mt = 0; mt < 2; ++mt)
          for (int h = 0; h < 2; ++h)
            tma_load_2d(smem + W_OFF + mt * kOperandTile + h * kOperandHalf, &tmW, w_full, h * 64, mt * 128);
        if (my_tiles > 0) issue_t(blockIdx.x, 0);          // first two t tiles in flight
        if (my_tiles > 1) issue_t(blockIdx.x + gridDim.x, 1);
      }
      __syncwarp();
      mbar_wait(w_full, 0, 20);
    }
    __syncwarp();
    for (int step = 0; step <= my_tiles; ++step) {
      if (warp == 0 && step < my_tiles) {
        const int acc = step & 1;
        mbar_wait(&acc_empty[acc], ((step >> 1) & 1) ^ 1, 21);
        mbar_wait(a1_full, step & 1, 22);
        mbar_wait(a2_full, step & 1, 23);
        tc_fence_after_sync();
        if (leader) {
          umma_k128(tmem_base + acc * 256, a1_s, w_s, idesc, false);                       // p_out(LN_out(t))
          umma_k128(tmem_base + acc * 256 + 128, a2_s, w_s + kOperandTile, idesc, false);  // g_out(LN_in(z))
          umma_commit(a_empty);
          umma_commit(&acc_full[acc]);
        }
        __syncwarp();
        if (step + 2 < my_tiles) {  // refill the raw-t stage this tile used, once the transformers have released it
          mbar_wait(&t_empty[step & 1], (step >> 1) & 1, 24);
          if (leader) issue_t(blockIdx.x + (step + 2) * gridDim.x, step & 1);
        }
      }
      __syncwarp();
      if (step == 0) continue;
      const int it = step - 1;
      const int tile = blockIdx.x + it * gridDim.x;
      const int line = tile / tiles_per_line;
      const int pos0 = (tile - line * tiles_per_line) << 7;
      const int acc = it & 1;
      const bool valid = (pos0 + r) < p.n_pos;
      const uint8_t* zrow = static_cast<const uint8_t*>(p.z) + line * p.z_line_stride + (pos0 + r) * p.z_pos_stride;
      mbar_wait(&acc_full[acc], (it >> 1) & 1, 28);
      tc_fence_after_sync();
      const uint32_t p_addr = tmem_addr(tmem_base, warp * 32, acc * 256);
      const uint32_t g_addr = p_addr + 128;
      uint32_t pa[16], ga[16], pb[16], gb[16];
      tmem_ld_32x16(p_addr, pa);
      tmem_ld_32x16(g_addr, ga);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint8_t* stage = smem + STAGE_OFF + ((c / CPS) & 1) * kOperandHalf;
        if (c % CPS == 0) {  // the store that last used this staging tile has finished reading it
          if (r == 0) tma_store_wait_read1();
          named_bar_sync(1, 128);
        }
        uint32_t(&pv)[16] = (c & 1) ? pb : pa;
        uint32_t(&gv)[16] = (c & 1) ? gb : ga;
        tmem_ld_wait();
        if (c < 7) {
          tmem_ld_32x16(p_addr + (c + 1) * 16, (c & 1) ? pa : pb);
          tmem_ld_32x16(g_addr + (c + 1) * 16, (c & 1) ? ga : gb);
        } else {
          tc_fence_before_sync();
          mbar_arrive(&acc_empty[acc]);
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float x[8];
          if (read_res && valid) {
            load8<F32>(zrow, c * 16 + g * 8, x);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = 0.f;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e)
            x[e] = fmaf(__uint_as_float(pv[g * 8 + e]), sigmoid_fast(__uint_as_float(gv[g * 8 + e])), x[e]);
          if (F32) {
            const int k = (c % CPS) * 4 + g * 2;
            *reinterpret_cast<float4*>(stage + sw128_offset(r, k)) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(stage + sw128_offset(r, k + 1)) = make_float4(x[4], x[5], x[6], x[7]);
          } else {
            *reinterpret_cast<uint4*>(stage + sw128_offset(r, (c % CPS) * 2 + g)) = make_uint4(
                pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
          }
        }
        if (c % CPS == CPS - 1) {
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (r == 0) {
            const int ch0 = (c / CPS) * (F32 ? 32 : 64);
            const int c1 = p.pos_is_dim1 ? pos0 : line, c2 = p.pos_is_dim1 ? line : pos0;
            if (reduce)
              tma_reduce_add_3d(&tmO, stage, ch0, c1, c2);
            else
              tma_store_3d(&tmO, stage, ch0, c1, c2);
            tma_store_commit();
          }
        }
      }
    }
    if (r == 0) tma_store_wait0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200
