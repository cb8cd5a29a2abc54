// C ABI of the library (declared in include/b200pair.h): argument checks, tensor-map
// construction and kernel launches.  The kernels live in the .cuh files beside this one and are
// compiled into this single translation unit.
#include <cstdarg>

#include "host_util.cuh"
#include "umma.cuh"
#include "row_tile.cuh"
#include "bmm_nt.cuh"
#include "trimul.cuh"
#include "transition.cuh"
#include "elementwise.cuh"
#include "opm.cuh"
#include "attention.cuh"
#include "pair_bias.cuh"
#include "triatt.cuh"
#include "window_attention.cuh"

namespace b200 {

template <class Kernel>
static int set_smem(Kernel k, uint32_t bytes) {
  return set_smem_once(reinterpret_cast<const void*>(k), bytes);
}

template <int DH>
static int launch_window_attention(const WindowAttnParams& p, int BM, cudaStream_t st) {
  const uint32_t smem = uint32_t(2u * p.Hk * p.heads * DH * 2u + p.Hk + 16);
  if (int e = set_smem(window_attention_kernel<DH>, smem)) return e;
  window_attention_kernel<DH><<<BM * p.NW, p.heads * p.W, smem, st>>>(p);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

struct BmmLaunch {
  const void* A;
  const void* B;
  void* C;
  int batch, M, N, K;
  int64_t lda, ldb, ldc, sa, sb, sc;  // elements
  float scale = 1.0f;
  const float* scale_ptr = nullptr;
  const float* bias = nullptr;
  int out_f32 = 0;
  int opm_ntok = 0;
  const void* residual = nullptr;
  int remap_n = 0, remap_m = 0;
};

static int launch_bmm(const BmmLaunch& a, cudaStream_t stream) {
  const int BN = (a.N % 256 == 0 || a.N > 1024) ? 256 : 128;
  CUtensorMap tmA, tmB;
  const bool a_shared = a.batch > 1 && a.sa == 0;  // one A for every batch item
  {
    const uint64_t dims[3] = {uint64_t(a.K), uint64_t(a.M), uint64_t(a_shared ? 1 : a.batch)};
    const uint64_t str[2] = {uint64_t(a.lda) * 2, uint64_t(a.sa > 0 ? a.sa : a.lda * a.M) * 2};
    const uint32_t box[3] = {64, 128, 1};
    if (int e = make_tmap_bf16(&tmA, a.A, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(a.K), uint64_t(a.N), uint64_t(a.batch)};
    const uint64_t str[2] = {uint64_t(a.ldb) * 2, uint64_t(a.sb > 0 ? a.sb : a.ldb * a.N) * 2};
    const uint32_t box[3] = {64, uint32_t(BN), 1};
    if (int e = make_tmap_bf16(&tmB, a.B, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  BmmParams p;
  p.C = a.C;
  p.c_batch_stride = a.sc;
  p.ldc = int(a.ldc);
  p.m_valid = a.M;
  p.n_valid = a.N;
  p.tiles_m = (a.M + 127) / 128;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.batch = a.batch;
  p.k_blocks = (a.K + 63) / 64;
  p.scale = a.scale;
  p.scale_ptr = a.scale_ptr;
  p.bias = a.bias;
  p.out_f32 = a.out_f32;
  p.opm_ntok = a.opm_ntok;
  p.residual = a.residual;
  p.remap_n = a.remap_n;
  p.remap_m = a.remap_m > 0 ? a.remap_m : a.remap_n;
  p.a_shared = a_shared ? 1 : 0;
  // Bulk output through the C tensor map where the layout allows it: whole 128-byte column groups, the
  // residual (if any) being C itself, and for the transposed pair store lines that are whole row tiles.
  p.tma_c = 0;
  CUtensorMap tmC = tmA;
  const int64_t c_batch = a.sc > 0 ? a.sc : a.ldc * int64_t(a.M);
  const int c_esz = a.out_f32 ? 4 : 2;
  const int c_cols = 128 / c_esz;  // columns of one staging tile
  if (a.opm_ntok == 0 && a.N % c_cols == 0 && (a.ldc * c_esz) % 16 == 0 && (c_batch * c_esz) % 16 == 0 && aligned(a.C, 16) &&
      (a.residual == nullptr || a.residual == a.C) && (a.bias == nullptr || aligned(a.bias, 16)) &&
      (a.remap_n == 0 || (a.remap_n % 128 == 0 && a.batch == 1 && a.M == a.remap_n * p.remap_m))) {
    uint64_t dims[3], str[2];
    uint32_t box[3];
    dims[0] = uint64_t(a.N);
    box[0] = uint32_t(c_cols);
    if (a.remap_n > 0) {  // {column, line, pos}: pair (line, pos) lives in row pos * remap_m + line
      dims[1] = uint64_t(p.remap_m), dims[2] = uint64_t(a.remap_n);
      str[0] = uint64_t(a.ldc) * c_esz, str[1] = uint64_t(a.ldc) * c_esz * uint64_t(p.remap_m);
      box[1] = 1, box[2] = 128;
    } else {
      dims[1] = uint64_t(a.M), dims[2] = uint64_t(a.batch);
      str[0] = uint64_t(a.ldc) * c_esz, str[1] = uint64_t(c_batch) * c_esz;
      box[1] = 128, box[2] = 1;
    }
    if (int e = make_tmap(&tmC, a.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.C, 3, dims,
                          str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
    p.tma_c = a.residual ? 2 : 1;
  }
  const int total = p.tiles_m * p.tiles_n * a.batch;
  const int grid = total < sm_count() ? total : sm_count();
  if (BN == 256) {
    if (int e = set_smem(bmm_nt_kernel<256>, BmmCfg<256>::SMEM_BYTES)) return e;
    bmm_nt_kernel<256><<<grid, 192, BmmCfg<256>::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  } else {
    if (int e = set_smem(bmm_nt_kernel<128>, BmmCfg<128>::SMEM_BYTES)) return e;
    bmm_nt_kernel<128><<<grid, 192, BmmCfg<128>::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  }
  B200_AFTER_LAUNCH();
  return 0;
}

static int launch_rows_to_bf16(const void* x, bool f32, __nv_bfloat16* y, const float* w, const float* b,
                               int64_t rows, int cols, bool normalize, cudaStream_t stream, bool silu = false,
                               const void* x2 = nullptr, int cols1 = 0) {
  const int warps = 8;
  int64_t blocks = (rows + warps - 1) / warps;
  const int64_t cap = int64_t(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (!x2 && cols <= 128) {  // narrow rows: several rows per warp
    const int nn = normalize, ss = silu;
    if (cols <= 64) {
      if (f32) layernorm_rows_narrow_kernel<true, 8><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, nn, ss);
      else layernorm_rows_narrow_kernel<false, 8><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, nn, ss);
    } else {
      if (f32) layernorm_rows_narrow_kernel<true, 16><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, nn, ss);
      else layernorm_rows_narrow_kernel<false, 16><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, nn, ss);
    }
    B200_AFTER_LAUNCH();
    return 0;
  }
  if (f32)
    layernorm_rows_kernel<true><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, normalize, silu,
                                                                       x2, cols1);
  else
    layernorm_rows_kernel<false><<<int(blocks), warps * 32, 0, stream>>>(x, y, w, b, rows, cols, 1e-5f, normalize, silu,
                                                                        x2, cols1);
  B200_AFTER_LAUNCH();
  return 0;
}

// Describes where the attention core finds its operands (all bf16, device memory).
struct FlashLaunch {
  const void* qk;        // rows of `qk_width` columns; Q heads at q_col0 + h*DH, K heads at k_col0 + h*DH
  int64_t qk_width;      // elements per row
  int64_t qk_b_stride;   // elements between batch items
  const void* vT;        // [Bt][H*DH][v_pitch]
  int64_t v_pitch;
  const void* bias;      // [groups*H][N][bias_pitch]
  int64_t bias_pitch;
  int bias_groups;
  FlashParams p;
};

template <int DH, int G>
static int launch_flash_t(const FlashLaunch& a, cudaStream_t stream) {
  using Cfg = FlashCfg<DH, G>;
  const FlashParams& p0 = a.p;
  CUtensorMap tmQ, tmV, tmB;
  {
    const uint64_t dims[3] = {uint64_t(a.qk_width), uint64_t(p0.N), uint64_t(p0.Bt)};
    const uint64_t str[2] = {uint64_t(a.qk_width) * 2, uint64_t(a.qk_b_stride) * 2};
    const uint32_t box[3] = {uint32_t(DH), 128, 1};
    if (int e = make_tmap_bf16(&tmQ, a.qk, 3, dims, str, box,
                               DH == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(p0.N), uint64_t(p0.H) * DH, uint64_t(p0.Bt)};
    const uint64_t str[2] = {uint64_t(a.v_pitch) * 2, uint64_t(a.v_pitch) * p0.H * DH * 2};
    const uint32_t box[3] = {64, uint32_t(DH), 1};
    if (int e = make_tmap_bf16(&tmV, a.vT, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(p0.N), uint64_t(p0.N), uint64_t(a.bias_groups) * p0.H};
    const uint64_t str[2] = {uint64_t(a.bias_pitch) * 2, uint64_t(a.bias_pitch) * p0.N * 2};
    const uint32_t box[3] = {64, 128, 1};
    if (int e = make_tmap_bf16(&tmB, a.bias, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  FlashParams p = p0;
  p.nqt = (p.N + 127) / 128;
  p.nkt = (p.N + 127) / 128;
  if (p.nkt > Cfg::MAX_T)
    return fail(B200_ERR_INVALID_ARGUMENT, "attention supports at most %d tokens (got %d)", Cfg::MAX_T * 128, p.N);
  p.nqg = (p.nqt + G - 1) / G;
  p.total_work = p.Bt * p.H * p.nqg;
  if (int e = set_smem(flash_core_kernel<DH, G>, Cfg::SMEM_BYTES)) return e;
  const int grid = p.total_work < sm_count() ? p.total_work : sm_count();
  flash_core_kernel<DH, G><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmQ, tmQ, tmV, tmB, p);
  B200_AFTER_LAUNCH();
  return 0;
}

static int launch_flash(const FlashLaunch& a, int DH, cudaStream_t stream) {
  return DH == 32 ? launch_flash_t<32, 2>(a, stream) : launch_flash_t<64, 1>(a, stream);
}

static int launch_pair_bias(const void* z, bool f32, const float* ln_w, const float* ln_b, const void* w_z,
                            __nv_bfloat16* zb, int n_lines, int n_pos, long long z_line_stride, long long z_pos_stride,
                            long long out_plane, long long out_pitch, int H, cudaStream_t stream) {
  CUtensorMap tmW;
  const uint64_t dims[2] = {128, 16};
  const uint64_t str[1] = {256};
  const uint32_t box[2] = {64, 16};
  if (int e = make_tmap_bf16(&tmW, w_z, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  if (int e = set_smem(pair_bias_kernel<true>, pair_bias::SMEM_BYTES)) return e;
  if (int e = set_smem(pair_bias_kernel<false>, pair_bias::SMEM_BYTES)) return e;
  PairBiasParams p;
  p.z = z;
  p.ln_w = ln_w;
  p.ln_b = ln_b;
  p.zb = zb;
  p.n_lines = n_lines;
  p.n_pos = n_pos;
  p.z_line_stride = z_line_stride;
  p.z_pos_stride = z_pos_stride;
  p.out_plane = out_plane;
  p.out_pitch = out_pitch;
  p.H = H;
  p.num_tiles = n_lines * ((n_pos + 127) / 128);
  p.scale = 1.4426950408889634f;
  p.eps = 1e-5f;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  if (f32)
    pair_bias_kernel<true><<<grid, pair_bias::THREADS, pair_bias::SMEM_BYTES, stream>>>(tmW, p);
  else
    pair_bias_kernel<false><<<grid, pair_bias::THREADS, pair_bias::SMEM_BYTES, stream>>>(tmW, p);
  B200_AFTER_LAUNCH();
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_version(void) { return 100; }

const char* b200_last_error(void) { return g_last_error; }

// Compute capability check only (cached per thread); *dev_out receives the current device ordinal.
static int check_arch(int* dev_out) {
  static thread_local int cached_dev = -1;
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev_out) *dev_out = dev;
  if (dev == cached_dev) return B200_OK;
  int major = 0;
  B200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return fail(B200_ERR_UNSUPPORTED_DEVICE, "device %d has compute capability %d.x; this library is sm_100a only",
                dev, major);
  cached_dev = dev;
  return B200_OK;
}

// Host-visible copy of the device status word, one per device ordinal: 64 bytes of pinned, mapped host memory
// that a kernel writes when one of its bounded waits runs out.  Set up by the first ordinary call on a device.
static int* g_host_status[64] = {nullptr};

static int ensure_host_status(int dev) {
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (g_host_status[dev]) return B200_OK;
  int* hp = nullptr;
  B200_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&hp), 64, cudaHostAllocMapped | cudaHostAllocPortable));
  *hp = 0;
  int* dp = nullptr;
  B200_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dp), hp, 0));
  B200_CUDA(cudaMemcpyToSymbol(g_host_status_ptr, &dp, sizeof(dp)));
  g_host_status[dev] = hp;
  return B200_OK;
}

int b200_check_device(void) {
  int dev = 0;
  if (int e = check_arch(&dev)) return e;
  if (dev < 0 || dev >= 64) return B200_OK;
  if (!g_host_status[dev])
    if (int e = ensure_host_status(dev)) return e;
  const int st = *reinterpret_cast<volatile int*>(g_host_status[dev]);
  if (st != 0)
    return fail(B200_ERR_DEVICE_WAIT,
                "an earlier kernel on device %d gave up a bounded wait (status %#x, wait site %d): its results and "
                "those of the kernels after it are invalid; b200_device_status() reads and clears the status",
                dev, st, st >> 8);
  return B200_OK;
}

int b200_peek_status(int* status) {
  B200_CHECK_ARG(status != nullptr, "status is NULL");
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  *status = (dev >= 0 && dev < 64 && g_host_status[dev]) ? *reinterpret_cast<volatile int*>(g_host_status[dev]) : 0;
  return B200_OK;
}

unsigned long long b200_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int b200_device_status(int* status) {
  B200_CHECK_ARG(status != nullptr, "status is NULL");
  B200_CUDA(cudaDeviceSynchronize());
  int v = 0;
  B200_CUDA(cudaMemcpyFromSymbol(&v, g_dev_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    B200_CUDA(cudaMemcpyToSymbol(g_dev_status, &zero, sizeof(int)));
  }
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && g_host_status[dev]) *reinterpret_cast<volatile int*>(g_host_status[dev]) = 0;
  *status = v;
  return B200_OK;
}

int b200_layernorm_fwd(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, float eps,
                       b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && y, "x/y is NULL");
  B200_CHECK_ARG(rows >= 0, "rows < 0");
  B200_CHECK_ARG(cols > 0 && cols % 8 == 0 && cols <= 1024, "cols=%d must be a multiple of 8 and <= 1024", cols);
  B200_CHECK_ARG(aligned(x, 16) && aligned(y, 16), "x/y must be 16-byte aligned");
  if (rows == 0) return B200_OK;
  const int warps = 8;
  int64_t blocks = (rows + warps - 1) / warps;
  const int64_t cap = int64_t(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  layernorm_rows_kernel<false><<<int(blocks), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<__nv_bfloat16*>(y), w, b, rows, cols, eps, 1, 0);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_bmm_nt_bf16(const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda,
                     int64_t ldb, int64_t ldc, int64_t sa, int64_t sb, int64_t sc, float scale,
                     b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(A && B && C, "A/B/C is NULL");
  B200_CHECK_ARG(batch > 0 && M > 0 && N > 0 && K > 0, "batch/M/N/K must be positive");
  B200_CHECK_ARG(N % 8 == 0, "N=%d must be a multiple of 8", N);
  B200_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "row pitches must be multiples of 8 elements");
  B200_CHECK_ARG(sa % 8 == 0 && sb % 8 == 0 && sc % 8 == 0, "batch strides must be multiples of 8 elements");
  B200_CHECK_ARG(batch == 1 || (sa > 0 && sb > 0), "batch strides must be positive");
  B200_CHECK_ARG(lda >= K && ldb >= K && ldc >= N, "row pitch smaller than the row");
  B200_CHECK_ARG(aligned(A, 16) && aligned(B, 16) && aligned(C, 16), "A/B/C must be 16-byte aligned");
  BmmLaunch a{A, B, C, batch, M, N, K, lda, ldb, ldc, sa, sb, sc};
  a.scale = scale;
  return launch_bmm(a, static_cast<cudaStream_t>(stream));
}

static inline int padded_n(int N) { return (N + 127) / 128 * 128; }

size_t b200_trimul_workspace_bytes(int N) {
  if (N <= 0) return 0;
  const size_t Np = size_t(padded_n(N));
  return 3 * size_t(kD) * Np * Np * sizeof(__nv_bfloat16);  // a, b, t
}

// Slab geometry of the two pair-walking kernels of triangle multiplication.
struct TriMulGeom {
  int n_lines, n_pos, lines_alloc, pos_pitch;
  long long z_line_stride, z_pos_stride;  // bytes
  long long m_line_stride, m_pos_stride;  // bytes
};

static int launch_trimul_project(const void* z, const uint8_t* mask, __nv_bfloat16* a_buf, __nv_bfloat16* b_buf,
                                 const b200_trimul_weights* w, const TriMulGeom& g, bool f32, cudaStream_t stream) {
  CUtensorMap tmWin;
  const uint64_t dims[2] = {128, 512};
  const uint64_t str[1] = {256};
  const uint32_t box[2] = {64, 128};
  if (int e = make_tmap_bf16(&tmWin, w->w_in, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  CUtensorMap tmA, tmB;  // channel-major a/b planes, stored as [128 channels][64 pairs] boxes of one line
  {
    const uint64_t dims[3] = {uint64_t(g.pos_pitch), uint64_t(g.lines_alloc), uint64_t(kD)};
    const uint64_t str[2] = {uint64_t(g.pos_pitch) * 2, uint64_t(g.pos_pitch) * g.lines_alloc * 2};
    const uint32_t box[3] = {64, 1, 128};
    if (int e = make_tmap_bf16(&tmA, a_buf, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    if (int e = make_tmap_bf16(&tmB, b_buf, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  if (int e = set_smem(trimul_in_kernel<true>, trimul_in::SMEM_BYTES)) return e;
  if (int e = set_smem(trimul_in_kernel<false>, trimul_in::SMEM_BYTES)) return e;
  TriMulInParams pi;
  pi.z = z;
  pi.mask = mask;
  pi.ln_w = w->ln_in_w;
  pi.ln_b = w->ln_in_b;
  pi.a_out = a_buf;
  pi.b_out = b_buf;
  pi.n_lines = g.n_lines;
  pi.n_pos = g.n_pos;
  pi.lines_alloc = g.lines_alloc;
  pi.pos_pitch = g.pos_pitch;
  pi.z_line_stride = g.z_line_stride;
  pi.z_pos_stride = g.z_pos_stride;
  pi.m_line_stride = g.m_line_stride;
  pi.m_pos_stride = g.m_pos_stride;
  pi.num_tiles = g.n_lines * (g.pos_pitch / 128);
  pi.eps = 1e-5f;
  const int grid = pi.num_tiles < sm_count() ? pi.num_tiles : sm_count();
  if (f32)
    trimul_in_kernel<true><<<grid, trimul_in::THREADS, trimul_in::SMEM_BYTES, stream>>>(tmWin, tmA, tmB, pi);
  else
    trimul_in_kernel<false><<<grid, trimul_in::THREADS, trimul_in::SMEM_BYTES, stream>>>(tmWin, tmA, tmB, pi);
  B200_AFTER_LAUNCH();
  return 0;
}

static int launch_trimul_output(const void* z, void* out, const __nv_bfloat16* t_buf, const b200_trimul_weights* w,
                                const TriMulGeom& g, bool add_residual, bool f32, cudaStream_t stream) {
  CUtensorMap tmWout, tmT;
  {
    const uint64_t dims[2] = {128, 256};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmWout, w->w_out, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(g.pos_pitch), uint64_t(g.lines_alloc), uint64_t(kD)};
    const uint64_t str[2] = {uint64_t(g.pos_pitch) * 2, uint64_t(g.pos_pitch) * g.lines_alloc * 2};
    const uint32_t box[3] = {128, 1, 128};
    if (int e = make_tmap_bf16(&tmT, t_buf, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
  }
  // Output tiles [128 pairs][128 B of channels]; the dimension with the smaller stride comes first.
  CUtensorMap tmO;
  const bool pos_first = g.z_pos_stride <= g.z_line_stride;
  {
    const uint64_t np = uint64_t(g.n_pos), nl = uint64_t(g.n_lines);
    const uint64_t dims[3] = {uint64_t(kD), pos_first ? np : nl, pos_first ? nl : np};
    const uint64_t str[2] = {uint64_t(pos_first ? g.z_pos_stride : g.z_line_stride),
                             uint64_t(pos_first ? g.z_line_stride : g.z_pos_stride)};
    const uint32_t box[3] = {f32 ? 32u : 64u, pos_first ? 128u : 1u, pos_first ? 1u : 128u};
    if (int e = make_tmap(&tmO, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, 3, dims,
                          str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  if (int e = set_smem(trimul_out_kernel<true>, trimul_out::SMEM_BYTES)) return e;
  if (int e = set_smem(trimul_out_kernel<false>, trimul_out::SMEM_BYTES)) return e;
  TriMulOutParams po;
  po.z = z;
  po.out = out;
  po.ln_in_w = w->ln_in_w;
  po.ln_in_b = w->ln_in_b;
  po.ln_out_w = w->ln_out_w;
  po.ln_out_b = w->ln_out_b;
  po.n_lines = g.n_lines;
  po.n_pos = g.n_pos;
  po.pos_pitch = g.pos_pitch;
  po.z_line_stride = g.z_line_stride;
  po.z_pos_stride = g.z_pos_stride;
  po.pos_is_dim1 = pos_first ? 1 : 0;
  po.num_tiles = g.n_lines * (g.pos_pitch / 128);
  po.add_residual = add_residual ? 1 : 0;
  po.eps = 1e-5f;
  const int grid = po.num_tiles < sm_count() ? po.num_tiles : sm_count();
  if (f32)
    trimul_out_kernel<true><<<grid, trimul_out::THREADS, trimul_out::SMEM_BYTES, stream>>>(tmWout, tmT, tmO, po);
  else
    trimul_out_kernel<false><<<grid, trimul_out::THREADS, trimul_out::SMEM_BYTES, stream>>>(tmWout, tmT, tmO, po);
  B200_AFTER_LAUNCH();
  return 0;
}

static bool trimul_weights_ok(const b200_trimul_weights* w) {
  return w && w->w_in && w->w_out && w->ln_in_w && w->ln_in_b && w->ln_out_w && w->ln_out_b && aligned(w->w_in, 16) &&
         aligned(w->w_out, 16);
}

// Argument checks and the three launches of triangle multiplication; the callers have checked the device.
static int trimul_fwd_impl(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                           int incoming, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                           b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(z && mask && out && w, "z/mask/out/w is NULL");
  B200_CHECK_ARG(trimul_weights_ok(w), "a weight pointer is NULL or not 16-byte aligned");
  B200_CHECK_ARG(B > 0 && N > 0, "B=%d, N=%d must be positive", B, N);
  B200_CHECK_ARG(z_dtype == B200_DTYPE_BF16 || z_dtype == B200_DTYPE_F32, "unknown z_dtype %d", z_dtype);
  B200_CHECK_ARG(aligned(z, 32) && aligned(out, 32), "z/out must be 32-byte aligned");
  const bool f32 = z_dtype == B200_DTYPE_F32;
  const size_t esz = f32 ? 4 : 2;
  const size_t need = b200_trimul_workspace_bytes(N);
  if (!workspace || workspace_bytes < need || !aligned(workspace, 1024))
    return fail(B200_ERR_WORKSPACE, "workspace must be 1024-byte aligned and hold %zu bytes (got %zu)", need,
                workspace_bytes);
  const int Np = padded_n(N);
  const size_t plane = size_t(kD) * Np * Np;
  __nv_bfloat16* a_buf = static_cast<__nv_bfloat16*>(workspace);
  __nv_bfloat16* b_buf = a_buf + plane;
  __nv_bfloat16* t_buf = b_buf + plane;
  const long long row_b = (long long)N * kD * esz, col_b = (long long)kD * esz;
  // projection walks rows (outgoing) or columns (incoming); the output stage always walks rows
  TriMulGeom gin{N, N, Np, Np, incoming ? col_b : row_b, incoming ? row_b : col_b, incoming ? 1 : N, incoming ? N : 1};
  TriMulGeom gout{N, N, Np, Np, row_b, col_b, 0, 0};
  for (int bi = 0; bi < B; ++bi) {
    const uint8_t* zb = static_cast<const uint8_t*>(z) + size_t(bi) * N * N * kD * esz;
    uint8_t* ob = static_cast<uint8_t*>(out) + size_t(bi) * N * N * kD * esz;
    if (int e = launch_trimul_project(zb, mask + size_t(bi) * N * N, a_buf, b_buf, w, gin, f32, stream)) return e;
    {
      const int64_t plane_el = int64_t(Np) * Np;
      BmmLaunch a{a_buf, b_buf, t_buf, kD, Np, Np, Np, Np, Np, Np, plane_el, plane_el, plane_el};
      if (int e = launch_bmm(a, stream)) return e;
    }
    if (int e = launch_trimul_output(zb, ob, t_buf, w, gout, add_residual != 0, f32, stream)) return e;
  }
  return B200_OK;
}

int b200_trimul_fwd(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                    int incoming, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                    b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  return trimul_fwd_impl(z, mask, out, w, B, N, incoming, add_residual, z_dtype, workspace, workspace_bytes, stream);
}

// Staged form for sharded callers: the projection and output stages on a rectangular slab, the contraction
// (b200_bmm_nt) and whatever exchange the caller needs in between.
int b200_trimul_project(const void* z, const uint8_t* mask, void* a_out, void* b_out, const b200_trimul_weights* w,
                        int n_rows, int n_cols, int64_t z_row_stride, int64_t mask_row_stride, int incoming,
                        int pos_pitch, int z_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(z && mask && a_out && b_out, "z/mask/a_out/b_out is NULL");
  B200_CHECK_ARG(trimul_weights_ok(w), "a weight pointer is NULL or not 16-byte aligned");
  B200_CHECK_ARG(n_rows > 0 && n_cols > 0, "n_rows=%d, n_cols=%d must be positive", n_rows, n_cols);
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown z_dtype %d", z_dtype);
  const int n_pos = incoming ? n_rows : n_cols, n_lines = incoming ? n_cols : n_rows;
  B200_CHECK_ARG(pos_pitch % 128 == 0 && pos_pitch >= n_pos, "pos_pitch=%d must be a multiple of 128 and >= %d", pos_pitch,
                 n_pos);
  B200_CHECK_ARG(z_row_stride >= int64_t(n_cols) * kD && z_row_stride % 8 == 0 && mask_row_stride >= n_cols,
                 "row strides smaller than a row");
  B200_CHECK_ARG(aligned(z, 32) && aligned(a_out, 16) && aligned(b_out, 16), "z must be 32-byte aligned, a/b 16-byte");
  const bool f32 = z_dtype == B200_DTYPE_F32;
  const long long esz = f32 ? 4 : 2;
  const long long row_b = z_row_stride * esz, col_b = kD * esz;
  TriMulGeom g{n_lines, n_pos, n_lines, pos_pitch, incoming ? col_b : row_b, incoming ? row_b : col_b,
               incoming ? 1 : mask_row_stride, incoming ? mask_row_stride : 1};
  return launch_trimul_project(z, mask, static_cast<__nv_bfloat16*>(a_out), static_cast<__nv_bfloat16*>(b_out), w, g, f32,
                               static_cast<cudaStream_t>(stream));
}

int b200_trimul_output(const void* t, const void* z, void* out, const b200_trimul_weights* w, int n_rows, int n_cols,
                       int64_t z_row_stride, int transposed_t, int pos_pitch, int add_residual, int z_dtype,
                       b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(t && z && out, "t/z/out is NULL");
  B200_CHECK_ARG(trimul_weights_ok(w), "a weight pointer is NULL or not 16-byte aligned");
  B200_CHECK_ARG(n_rows > 0 && n_cols > 0, "n_rows=%d, n_cols=%d must be positive", n_rows, n_cols);
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown z_dtype %d", z_dtype);
  const int n_pos = transposed_t ? n_rows : n_cols, n_lines = transposed_t ? n_cols : n_rows;
  B200_CHECK_ARG(pos_pitch % 128 == 0 && pos_pitch >= n_pos, "pos_pitch=%d must be a multiple of 128 and >= %d", pos_pitch,
                 n_pos);
  B200_CHECK_ARG(z_row_stride >= int64_t(n_cols) * kD && z_row_stride % 8 == 0, "row stride smaller than a row");
  B200_CHECK_ARG(aligned(z, 32) && aligned(out, 32) && aligned(t, 16), "z/out must be 32-byte aligned, t 16-byte");
  const bool f32 = z_dtype == B200_DTYPE_F32;
  const long long esz = f32 ? 4 : 2;
  const long long row_b = z_row_stride * esz, col_b = kD * esz;
  TriMulGeom g{n_lines, n_pos, n_lines, pos_pitch, transposed_t ? col_b : row_b, transposed_t ? row_b : col_b, 0, 0};
  return launch_trimul_output(z, out, static_cast<const __nv_bfloat16*>(t), w, g, add_residual != 0, f32,
                              static_cast<cudaStream_t>(stream));
}

int b200_bmm_nt(const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda, int64_t ldb,
                int64_t ldc, int64_t a_batch_stride, int64_t b_batch_stride, int64_t c_batch_stride, float scale,
                int out_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(A && B && C, "A/B/C is NULL");
  B200_CHECK_ARG(batch > 0 && M > 0 && N > 0 && K > 0, "batch/M/N/K must be positive");
  B200_CHECK_ARG(N % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "N and the row pitches must be multiples of 8");
  B200_CHECK_ARG(a_batch_stride % 8 == 0 && b_batch_stride % 8 == 0 && c_batch_stride % 8 == 0,
                 "batch strides must be multiples of 8 elements");
  B200_CHECK_ARG(batch == 1 || (a_batch_stride >= 0 && b_batch_stride > 0),
                 "batch strides must be positive (a_batch_stride may be 0: one A shared by every batch item)");
  B200_CHECK_ARG(lda >= K && ldb >= K && ldc >= N, "row pitch smaller than the row");
  B200_CHECK_ARG((out_dtype | 1) == 1, "unknown out_dtype %d", out_dtype);
  B200_CHECK_ARG(aligned(A, 16) && aligned(B, 16) && aligned(C, 32), "A/B must be 16-byte aligned, C 32-byte aligned");
  BmmLaunch a{A, B, C, batch, M, N, K, lda, ldb, ldc, a_batch_stride, b_batch_stride, c_batch_stride};
  a.scale = scale;
  a.out_f32 = out_dtype == B200_DTYPE_F32;
  return launch_bmm(a, static_cast<cudaStream_t>(stream));
}

int b200_transition_fwd(const void* x, void* out, const void* w13, const void* w3, const float* ln_w,
                        const float* ln_b, int64_t rows, int use_norm, int add_residual, int x_dtype,
                        b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(x && out && w13 && w3, "x/out/w13/w3 is NULL");
  B200_CHECK_ARG(!use_norm || (ln_w && ln_b), "use_norm needs ln_w and ln_b");
  B200_CHECK_ARG(rows >= 0 && rows < (int64_t(1) << 31), "rows out of range");
  B200_CHECK_ARG(x_dtype == B200_DTYPE_BF16 || x_dtype == B200_DTYPE_F32, "unknown x_dtype %d", x_dtype);
  B200_CHECK_ARG(aligned(x, 32) && aligned(out, 32) && aligned(w13, 16) && aligned(w3, 16),
                 "x/out must be 32-byte aligned, weights 16-byte aligned");
  if (rows == 0) return B200_OK;
  CUtensorMap tmW1, tmW3;
  {
    const uint64_t dims[2] = {128, 1024};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmW1, w13, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[2] = {512, 128};
    const uint64_t str[1] = {1024};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmW3, w3, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  const bool tr_f32 = x_dtype == B200_DTYPE_F32;
  CUtensorMap tmO;  // output rows, [128 rows][64 B] boxes
  {
    const uint64_t dims[2] = {uint64_t(kD), uint64_t(rows)};
    const uint64_t str[1] = {uint64_t(kD) * (tr_f32 ? 4 : 2)};
    const uint32_t box[2] = {tr_f32 ? 16u : 32u, 128};
    if (int e = make_tmap(&tmO, tr_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, 2, dims, str,
                          box, CU_TENSOR_MAP_SWIZZLE_64B))
      return e;
  }
  if (int e = set_smem(transition_kernel<true>, transition::SMEM_BYTES)) return e;
  if (int e = set_smem(transition_kernel<false>, transition::SMEM_BYTES)) return e;
  TransitionParams p;
  p.x = x;
  p.out = out;
  p.ln_w = use_norm ? ln_w : nullptr;
  p.ln_b = use_norm ? ln_b : nullptr;
  p.rows = rows;
  p.num_tiles = int((rows + 127) / 128);
  p.use_norm = use_norm ? 1 : 0;
  p.add_residual = add_residual ? 1 : 0;
  p.eps = 1e-5f;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  if (x_dtype == B200_DTYPE_F32)
    transition_kernel<true><<<grid, transition::THREADS, transition::SMEM_BYTES, stream>>>(tmW1, tmW3, tmO, p);
  else
    transition_kernel<false><<<grid, transition::THREADS, transition::SMEM_BYTES, stream>>>(tmW1, tmW3, tmO, p);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// Scratch for b200_trimul_fwd_static: the three channel-major planes a, b, t for N <= 256 (padded to 256),
// plus slack so the base can be rounded up to the 1024-byte alignment the kernels' launcher asks for.
// It lives in the library image: every GPU that loads the library holds these 48 MiB until the process exits.
#define B200_STATIC_TRIMUL_MAX_N 256
static __device__ __align__(256) unsigned char g_trimul_static_scratch[size_t(3) * 128 * 256 * 256 * 2 + 1024];

// Device address of the scratch per device ordinal, resolved on first use with that device current.
// (In host code the array's name is only a handle for the runtime, never a pointer a kernel may be given.)
static void* g_trimul_static_ptr[64] = {nullptr};

int b200_trimul_fwd_static(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                           int incoming, int add_residual, int z_dtype, b200_stream_t stream) {
  // Only the compute-capability check: the ordinary entry points also set up a pinned status word on their first
  // call, which is an allocation this entry point promises not to make.
  if (int e = check_arch(nullptr)) return e;
  B200_CHECK_ARG(N > 0 && N <= B200_STATIC_TRIMUL_MAX_N,
                 "b200_trimul_fwd_static handles N <= %d (got %d); use b200_trimul_fwd with a caller workspace",
                 B200_STATIC_TRIMUL_MAX_N, N);
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CHECK_ARG(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (!g_trimul_static_ptr[dev]) {
    void* ptr = nullptr;
    B200_CUDA(cudaGetSymbolAddress(&ptr, g_trimul_static_scratch));
    g_trimul_static_ptr[dev] = ptr;
  }
  uintptr_t base = (reinterpret_cast<uintptr_t>(g_trimul_static_ptr[dev]) + 1023) & ~uintptr_t(1023);
  return trimul_fwd_impl(z, mask, out, w, B, N, incoming, add_residual, z_dtype, reinterpret_cast<void*>(base),
                         b200_trimul_workspace_bytes(N), stream);
}

// ------------------------------------------------------------------------------------------------ OPM
static void opm_plan(int S, int N, int* Sp, int* CI, size_t* ab_bytes, size_t* outer_bytes) {
  *Sp = (S + 7) / 8 * 8;
  const size_t per_tok = size_t(N) * 1024 * 2;               // bytes of outer products for one token row
  // Chunks near 1 GiB: an L2-sized chunk (48 MB) was measured slower, 0.58 ms against 0.42 ms for a 1024 x 384 MSA
  // (five times the launches, each with a tail).
  size_t ci = (size_t(1) << 30) / per_tok;
  ci = ci / 4 * 4;
  if (ci < 4) ci = 4;
  const size_t n4 = size_t(N + 3) / 4 * 4;
  if (ci > n4) ci = n4;
  *CI = int(ci);
  *ab_bytes = (size_t(N) * 32 * size_t(*Sp) * 2 + 1023) / 1024 * 1024;
  *outer_bytes = (ci * per_tok + 1023) / 1024 * 1024;
}

size_t b200_opm_workspace_bytes(int S, int N) {
  if (S <= 0 || N <= 0) return 0;
  int Sp, CI;
  size_t ab, outer;
  opm_plan(S, N, &Sp, &CI, &ab, &outer);
  return 2 * ab + outer + 1024;
}

// j0, nj: the token columns of the output to compute (all N rows always); ext_scale: device scalar replacing
// 1 / (number of valid MSA rows) -- for a caller that holds only part of the MSA depth; add_bias: whether proj_o's bias
// is added (exactly one of the partial results that are later summed should carry it).
static int opm_run(const void* m, const uint8_t* mask, int mask_ndim, void* out, const b200_opm_weights* w, int B,
                   int S, int N, int j0, int nj, const float* ext_scale, bool add_bias, int m_dtype, int out_dtype,
                   void* workspace, size_t workspace_bytes, b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(m && mask && out && w, "m/mask/out/w is NULL");
  B200_CHECK_ARG(w->w_ab && w->w_o && w->ln_w && w->ln_b && w->bias_o, "a weight pointer is NULL");
  B200_CHECK_ARG(B > 0 && S > 0 && N > 0, "B=%d, S=%d, N=%d must be positive", B, S, N);
  B200_CHECK_ARG(mask_ndim == 3 || (mask_ndim == 2 && B == 1), "mask must be [B,S,N], or [B,N] with B == 1");
  B200_CHECK_ARG((m_dtype | 1) == 1 && (out_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(m, 32) && aligned(out, 32) && aligned(w->w_ab, 16) && aligned(w->w_o, 16),
                 "m/out must be 32-byte aligned, weights 16-byte aligned");
  const size_t need = b200_opm_workspace_bytes(S, N);
  if (!workspace || workspace_bytes < need || !aligned(workspace, 1024))
    return fail(B200_ERR_WORKSPACE, "workspace must be 1024-byte aligned and hold %zu bytes (got %zu)", need,
                workspace_bytes);
  int Sp, CI;
  size_t ab_bytes, outer_bytes;
  opm_plan(S, N, &Sp, &CI, &ab_bytes, &outer_bytes);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* aT = reinterpret_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* bT = reinterpret_cast<__nv_bfloat16*>(ws + ab_bytes);
  __nv_bfloat16* outer = reinterpret_cast<__nv_bfloat16*>(ws + 2 * ab_bytes);
  float* inv = reinterpret_cast<float*>(ws + 2 * ab_bytes + outer_bytes);

  CUtensorMap tmW;
  {
    const uint64_t dims[2] = {64, 64};
    const uint64_t str[1] = {128};
    const uint32_t box[2] = {64, 64};
    if (int e = make_tmap_bf16(&tmW, w->w_ab, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  if (int e = set_smem(opm_proj_kernel<true>, opm_proj::SMEM_BYTES)) return e;
  if (int e = set_smem(opm_proj_kernel<false>, opm_proj::SMEM_BYTES)) return e;
  const size_t m_esz = m_dtype == B200_DTYPE_F32 ? 4 : 2;
  const size_t o_esz = out_dtype == B200_DTYPE_F32 ? 4 : 2;

  for (int bi = 0; bi < B; ++bi) {
    OpmProjParams pp;
    pp.m = static_cast<const uint8_t*>(m) + size_t(bi) * S * N * 64 * m_esz;
    pp.mask = mask + (mask_ndim == 3 ? size_t(bi) * S * N : 0);
    pp.mask_s_stride = mask_ndim == 3 ? N : 0;
    pp.ln_w = w->ln_w;
    pp.ln_b = w->ln_b;
    pp.aT = aT;
    pp.bT = bT;
    pp.S = S;
    pp.N = N;
    pp.Sp = Sp;
    pp.num_tiles = N * ((S + 127) / 128);
    pp.eps = 1e-5f;
    const int grid = pp.num_tiles < sm_count() ? pp.num_tiles : sm_count();
    if (m_dtype == B200_DTYPE_F32)
      opm_proj_kernel<true><<<grid, opm_proj::THREADS, opm_proj::SMEM_BYTES, stream>>>(tmW, pp);
    else
      opm_proj_kernel<false><<<grid, opm_proj::THREADS, opm_proj::SMEM_BYTES, stream>>>(tmW, pp);
    B200_AFTER_LAUNCH();
    const float* scale_ptr = ext_scale;
    if (mask_ndim == 3 && !ext_scale) {
      opm_inv_row_count_kernel<<<1, 1024, 0, stream>>>(pp.mask, S, N, inv);
      B200_AFTER_LAUNCH();
      scale_ptr = inv;
    }
    for (int i0 = 0; i0 < N; i0 += CI) {
      const int ci = (N - i0) < CI ? (N - i0) : CI;
      {
        BmmLaunch a{aT + size_t(i0) * 32 * Sp, bT + size_t(j0) * 32 * Sp, outer, 1, ci * 32, nj * 32, S, Sp, Sp, 0, 0, 0, 0};
        a.scale_ptr = scale_ptr;
        a.opm_ntok = nj;
        if (int e = launch_bmm(a, stream)) return e;
      }
      {
        void* dst = static_cast<uint8_t*>(out) + (size_t(bi) * N * nj + size_t(i0) * nj) * 128 * o_esz;
        BmmLaunch a{outer, w->w_o, dst, 1, ci * nj, 128, 1024, 1024, 1024, 128, 0, 0, 0};
        a.bias = add_bias ? w->bias_o : nullptr;
        a.out_f32 = out_dtype == B200_DTYPE_F32;
        if (int e = launch_bmm(a, stream)) return e;
      }
    }
  }
  return B200_OK;
}

int b200_opm_fwd(const void* m, const uint8_t* mask, int mask_ndim, void* out, const b200_opm_weights* w, int B,
                 int S, int N, int m_dtype, int out_dtype, void* workspace, size_t workspace_bytes,
                 b200_stream_t stream) {
  return opm_run(m, mask, mask_ndim, out, w, B, S, N, 0, N, nullptr, true, m_dtype, out_dtype, workspace, workspace_bytes,
                 stream);
}

int b200_opm_cols_fwd(const void* m, const uint8_t* mask, void* out, const b200_opm_weights* w, int S, int N, int j0,
                      int nj, const float* scale, int add_bias, int m_dtype, int out_dtype, void* workspace,
                      size_t workspace_bytes, b200_stream_t stream) {
  if (j0 < 0 || nj <= 0 || j0 + nj > N) return fail(B200_ERR_INVALID_ARGUMENT, "column range [%d, %d) outside [0, %d)", j0, j0 + nj, N);
  if (!scale) return fail(B200_ERR_INVALID_ARGUMENT, "scale is NULL");
  return opm_run(m, mask, 3, out, w, 1, S, N, j0, nj, scale, add_bias != 0, m_dtype, out_dtype, workspace, workspace_bytes,
                 stream);
}

// ------------------------------------------------------------------------------------------------ attention core
int b200_attention_core_fwd(const b200_attention_core_args* a, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(a != nullptr, "args is NULL");
  B200_CHECK_ARG(a->qk && a->vT && a->bias && a->mask && a->out, "qk/vT/bias/mask/out is NULL");
  B200_CHECK_ARG(a->head_dim_padded == 32 || a->head_dim_padded == 64, "head_dim_padded must be 32 or 64");
  B200_CHECK_ARG(a->N > 0 && a->H > 0 && a->batch > 0, "N/H/batch must be positive");
  B200_CHECK_ARG(a->head_dim_out > 0 && a->head_dim_out % 8 == 0 && a->head_dim_out <= a->head_dim_padded,
                 "head_dim_out must be a multiple of 8 and <= head_dim_padded");
  B200_CHECK_ARG(a->qk_width % 8 == 0 && a->v_pitch % 8 == 0 && a->bias_pitch % 8 == 0 && a->out_pitch % 8 == 0 &&
                     a->q_col0 % 8 == 0 && a->k_col0 % 8 == 0 && a->out_col0 % 8 == 0 && a->gate_col0 % 8 == 0 &&
                     a->gate_pitch % 8 == 0,
                 "pitches and column offsets must be multiples of 8 elements");
  B200_CHECK_ARG(a->bias_div > 0 && a->mask_div > 0 && a->bias_groups > 0, "bias_div/mask_div/bias_groups must be positive");
  B200_CHECK_ARG(aligned(a->qk, 16) && aligned(a->vT, 16) && aligned(a->bias, 16) && aligned(a->out, 16) &&
                     (!a->gate || aligned(a->gate, 16)), "operands must be 16-byte aligned");
  FlashLaunch l;
  l.qk = a->qk;
  l.qk_width = a->qk_width;
  l.qk_b_stride = a->qk_batch_stride;
  l.vT = a->vT;
  l.v_pitch = a->v_pitch;
  l.bias = a->bias;
  l.bias_pitch = a->bias_pitch;
  l.bias_groups = a->bias_groups;
  FlashParams& p = l.p;
  p.mask = a->mask;
  p.mask_div = a->mask_div;
  p.mask_row_stride = a->mask_row_stride;
  p.mask_key_stride = a->mask_key_stride;
  p.bias_div = a->bias_div;
  p.gate = static_cast<const __nv_bfloat16*>(a->gate);
  p.gate_activated = 0;
  p.gate_b_stride = a->gate_batch_stride;
  p.gate_pitch = a->gate_pitch;
  p.gate_col0 = a->gate_col0;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.out_b_stride = a->out_batch_stride;
  p.out_pitch = a->out_pitch;
  p.out_col0 = a->out_col0;
  p.dh_out = a->head_dim_out;
  p.N = a->N;
  p.H = a->H;
  p.Bt = a->batch;
  p.q_col0 = a->q_col0;
  p.k_col0 = a->k_col0;
  p.v_row0 = 0;
  return launch_flash(l, a->head_dim_padded, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------ APB
struct ApbPlan {
  int dh, DH, W1, Nk;
  size_t off_sln, off_qkg, off_vT, off_zb, off_og, total;
};

static bool apb_plan(int B, int M, int N, int c_s, int H, ApbPlan* pl) {
  if (H <= 0 || H > 16 || c_s % H != 0) return false;
  pl->dh = c_s / H;
  if (pl->dh % 8 != 0 || pl->dh > 64 || c_s % 8 != 0) return false;
  pl->DH = pl->dh <= 32 ? 32 : 64;
  pl->W1 = 2 * H * pl->DH + c_s;
  pl->Nk = (N + 7) / 8 * 8;
  const size_t rows = size_t(B) * M * N;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  size_t o = 0;
  pl->off_sln = o; o += up(rows * c_s * 2);
  pl->off_qkg = o; o += up(rows * pl->W1 * 2);
  pl->off_vT = o;  o += up(size_t(B) * M * H * pl->DH * pl->Nk * 2);
  pl->off_zb = o;  o += up(size_t(B) * H * N * pl->Nk * 2);
  pl->off_og = o;  o += up(rows * c_s * 2);
  pl->total = o;
  return true;
}

size_t b200_apb_workspace_bytes(int B, int M, int N, int c_s, int H) {
  ApbPlan pl;
  if (B <= 0 || M <= 0 || N <= 0 || !apb_plan(B, M, N, c_s, H, &pl)) return 0;
  return pl.total;
}

static int apb_run(const void* s, const void* z, const void* ext_bias, int64_t ext_bias_pitch, const uint8_t* mask,
                   void* out, const b200_apb_weights* w, int B, int M, int N, int c_s, int H, int s_dtype, int z_dtype,
                   void* workspace, size_t workspace_bytes, b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(s && (z || ext_bias) && mask && out && w, "s/z/mask/out/w is NULL");
  B200_CHECK_ARG(w->w_qkg && w->b_qkg && w->w_v && w->w_z && w->ln_z_w && w->w_o, "a weight pointer is NULL");
  B200_CHECK_ARG(B > 0 && M > 0 && N > 0, "B=%d, M=%d, N=%d must be positive", B, M, N);
  B200_CHECK_ARG((s_dtype | 1) == 1 && (z_dtype | 1) == 1, "unknown dtype");
  ApbPlan pl;
  B200_CHECK_ARG(apb_plan(B, M, N, c_s, H, &pl),
                 "unsupported c_s=%d, H=%d: need H <= 16, head dim a multiple of 8 and <= 64", c_s, H);
  B200_CHECK_ARG(aligned(s, 32) && (!z || aligned(z, 32)) && aligned(out, 32), "s/z/out must be 32-byte aligned");
  B200_CHECK_ARG(!ext_bias || (aligned(ext_bias, 16) && ext_bias_pitch % 8 == 0 && ext_bias_pitch >= N),
                 "bias must be 16-byte aligned with a pitch that is a multiple of 8 and >= N");
  if (!workspace || workspace_bytes < pl.total || !aligned(workspace, 1024))
    return fail(B200_ERR_WORKSPACE, "workspace must be 1024-byte aligned and hold %zu bytes (got %zu)", pl.total,
                workspace_bytes);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* s_ln = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_sln);
  __nv_bfloat16* qkg = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_qkg);
  __nv_bfloat16* vT = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_vT);
  __nv_bfloat16* zb = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_zb);
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_og);
  const int BM = B * M;
  const int64_t rows = int64_t(BM) * N;
  const int HD = H * pl.DH;

  // 1. LayerNorm (or plain conversion) of the single track
  if (int e = launch_rows_to_bf16(s, s_dtype == B200_DTYPE_F32, s_ln, w->ln_s_w, w->ln_s_b, rows, c_s,
                                  w->ln_s_w != nullptr, stream))
    return e;
  // 2. q | k | g projection (heads padded to DH, q pre-scaled) and V^T per batch item
  {
    BmmLaunch a{s_ln, w->w_qkg, qkg, 1, int(rows), pl.W1, c_s, c_s, c_s, pl.W1, 0, 0, 0};
    a.bias = w->b_qkg;
    if (int e = launch_bmm(a, stream)) return e;
  }
  for (int b = 0; b < BM; ++b) {
    BmmLaunch a{w->w_v, s_ln + size_t(b) * N * c_s, vT + size_t(b) * HD * pl.Nk, 1, HD, N, c_s, c_s, c_s, pl.Nk, 0, 0, 0};
    if (int e = launch_bmm(a, stream)) return e;
  }
  // 3. pair bias, one pass over z per batch element (unless the caller supplies it)
  const size_t z_esz = z_dtype == B200_DTYPE_F32 ? 4 : 2;
  for (int b = 0; b < B && !ext_bias; ++b) {
    if (int e = launch_pair_bias(static_cast<const uint8_t*>(z) + size_t(b) * N * N * kD * z_esz,
                                 z_dtype == B200_DTYPE_F32, w->ln_z_w, w->ln_z_b, w->w_z,
                                 zb + size_t(b) * H * N * pl.Nk, N, N, (long long)N * kD * z_esz, (long long)kD * z_esz,
                                 (long long)N * pl.Nk, pl.Nk, H, stream))
      return e;
  }
  // 4. attention core
  {
    FlashLaunch a;
    a.qk = qkg;
    a.qk_width = pl.W1;
    a.qk_b_stride = int64_t(N) * pl.W1;
    a.vT = vT;
    a.v_pitch = pl.Nk;
    a.bias = ext_bias ? ext_bias : static_cast<const void*>(zb);
    a.bias_pitch = ext_bias ? ext_bias_pitch : pl.Nk;
    a.bias_groups = B;
    FlashParams& p = a.p;
    p.mask = mask;
    p.mask_div = M;
    p.mask_row_stride = N;
    p.mask_key_stride = 1;
    p.bias_div = M;
    p.gate = qkg;
    p.gate_activated = 0;
    p.gate_b_stride = int64_t(N) * pl.W1;
    p.gate_pitch = pl.W1;
    p.gate_col0 = 2 * HD;
    p.out = og;
    p.out_b_stride = int64_t(N) * c_s;
    p.out_pitch = c_s;
    p.out_col0 = 0;
    p.dh_out = pl.dh;
    p.N = N;
    p.H = H;
    p.Bt = BM;
    p.q_col0 = 0;
    p.k_col0 = HD;
    p.v_row0 = 0;
    if (int e = launch_flash(a, pl.DH, stream)) return e;
  }
  // 5. output projection
  {
    BmmLaunch a{og, w->w_o, out, 1, int(rows), c_s, c_s, c_s, c_s, c_s, 0, 0, 0};
    a.out_f32 = s_dtype == B200_DTYPE_F32;
    if (int e = launch_bmm(a, stream)) return e;
  }
  return B200_OK;
}

int b200_apb_fwd(const void* s, const void* z, const uint8_t* mask, void* out, const b200_apb_weights* w, int B,
                 int M, int N, int c_s, int H, int s_dtype, int z_dtype, void* workspace, size_t workspace_bytes,
                 b200_stream_t stream) {
  if (!z) return fail(B200_ERR_INVALID_ARGUMENT, "z is NULL");
  return apb_run(s, z, nullptr, 0, mask, out, w, B, M, N, c_s, H, s_dtype, z_dtype, workspace, workspace_bytes, stream);
}

int b200_apb_fwd_bias(const void* s, const void* bias, int64_t bias_pitch, const uint8_t* mask, void* out,
                      const b200_apb_weights* w, int B, int M, int N, int c_s, int H, int s_dtype, void* workspace,
                      size_t workspace_bytes, b200_stream_t stream) {
  if (!bias) return fail(B200_ERR_INVALID_ARGUMENT, "bias is NULL");
  return apb_run(s, nullptr, bias, bias_pitch, mask, out, w, B, M, N, c_s, H, s_dtype, B200_DTYPE_F32, workspace,
                 workspace_bytes, stream);
}

int b200_pair_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w_z, void* out, int n_rows,
                       int n_cols, int64_t z_row_stride, int64_t out_plane, int64_t out_pitch, int H, int transposed,
                       int z_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(z && ln_w && w_z && out, "z/ln_w/w_z/out is NULL");
  B200_CHECK_ARG(n_rows > 0 && n_cols > 0 && H > 0 && H <= 16, "n_rows/n_cols must be positive, 1 <= H <= 16");
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown z_dtype %d", z_dtype);
  B200_CHECK_ARG(z_row_stride >= int64_t(n_cols) * kD && z_row_stride % 8 == 0, "row stride smaller than a row");
  const int n_lines = transposed ? n_cols : n_rows, n_pos = transposed ? n_rows : n_cols;
  B200_CHECK_ARG(out_pitch >= n_pos && out_plane >= int64_t(n_lines) * out_pitch, "output pitch/plane too small");
  B200_CHECK_ARG(aligned(z, 32) && aligned(w_z, 16), "z must be 32-byte aligned, w_z 16-byte aligned");
  const long long esz = z_dtype == B200_DTYPE_F32 ? 4 : 2;
  const long long row_b = z_row_stride * esz, col_b = kD * esz;
  return launch_pair_bias(z, z_dtype == B200_DTYPE_F32, ln_w, ln_b, w_z, static_cast<__nv_bfloat16*>(out), n_lines, n_pos,
                          transposed ? col_b : row_b, transposed ? row_b : col_b, out_plane, out_pitch, H,
                          static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------ triangle attention
// A slab holds `lines` complete attention rows: for the starting node a line is a row of z (the slab must span all
// columns), for the ending node a line is a column (the slab must span all rows); `pos` is the token axis attended over.
struct TriAttPlan {
  int lines, pos, Nk;
  size_t off_qkg, off_vT, off_tb, off_og, total;
};

static void triatt_plan(int lines, int pos, bool own_bias, TriAttPlan* pl) {
  pl->lines = lines;
  pl->pos = pos;
  pl->Nk = (pos + 7) / 8 * 8;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  size_t o = 0;
  pl->off_qkg = o; o += up(size_t(lines) * pos * 384 * 2);
  pl->off_vT = o;  o += up(size_t(lines) * kD * pl->Nk * 2);
  pl->off_tb = o;  o += own_bias ? up(size_t(4) * pos * pl->Nk * 2) : 0;
  pl->off_og = o;  o += up(size_t(lines) * pos * kD * 2);
  pl->total = o;
}

static int triatt_slab(const void* z, const uint8_t* mask, const void* ext_bias, int64_t ext_bias_pitch, void* out,
                       const b200_triatt_weights* w, int n_rows, int n_cols, bool ending, bool add_residual, bool f32,
                       void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const int lines = ending ? n_cols : n_rows, pos = ending ? n_rows : n_cols;
  TriAttPlan pl;
  triatt_plan(lines, pos, ext_bias == nullptr, &pl);
  if (!workspace || workspace_bytes < pl.total || !aligned(workspace, 1024))
    return fail(B200_ERR_WORKSPACE, "workspace must be 1024-byte aligned and hold %zu bytes (got %zu)", pl.total,
                workspace_bytes);
  if (!ext_bias && n_rows != n_cols)
    return fail(B200_ERR_INVALID_ARGUMENT, "a rectangular slab needs the triangle bias of the whole pair tensor");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* qkg = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_qkg);
  __nv_bfloat16* vT = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_vT);
  __nv_bfloat16* tb = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_tb);
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(ws + pl.off_og);
  const long long esz = f32 ? 4 : 2;
  const long long row_b = (long long)n_cols * kD * esz, col_b = kD * esz;
  const long long line_b = ending ? col_b : row_b, pos_b = ending ? row_b : col_b;

  CUtensorMap tmW;
  {
    const uint64_t dims[2] = {128, 512};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmW, w->w_qkgv, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  CUtensorMap tmQKG, tmVT;  // [128 rows][64 values] boxes: pairs x channels of q|k|g, channels x keys of V^T
  {
    const uint64_t dims[3] = {384, uint64_t(pos), uint64_t(lines)};
    const uint64_t str[2] = {768, uint64_t(pos) * 768};
    const uint32_t box[3] = {64, 128, 1};
    if (int e = make_tmap_bf16(&tmQKG, qkg, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(pos), uint64_t(kD), uint64_t(lines)};
    const uint64_t str[2] = {uint64_t(pl.Nk) * 2, uint64_t(pl.Nk) * kD * 2};
    const uint32_t box[3] = {64, 128, 1};
    if (int e = make_tmap_bf16(&tmVT, vT, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  CUtensorMap tmWB;  // the 8 rows of the bias weights that hold the 4 heads, as two 64-channel halves
  {
    const uint64_t dims[2] = {128, 16};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 8};
    if (int e = make_tmap_bf16(&tmWB, w->w_b, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  if (int e = set_smem(triatt_proj_kernel<true>, triatt_proj::SMEM_BYTES)) return e;
  if (int e = set_smem(triatt_proj_kernel<false>, triatt_proj::SMEM_BYTES)) return e;
  TriAttProjParams pp;
  pp.z = z;
  pp.ln_w = w->ln_w;
  pp.ln_b = w->ln_b;
  pp.g_bias = w->g_bias;
  pp.qkg = qkg;
  pp.vT = vT;
  pp.n_lines = lines;
  pp.n_pos = pos;
  pp.Nk = pl.Nk;
  pp.z_line_stride = line_b;
  pp.z_pos_stride = pos_b;
  pp.num_tiles = lines * ((pos + 127) / 128);
  pp.eps = 1e-5f;
  // Without a bias from the caller the projection kernel writes the triangle bias of the same rows itself.
  pp.tri_bias = ext_bias ? nullptr : tb;
  pp.bias_plane = (long long)pos * pl.Nk;
  pp.bias_pitch = pl.Nk;
  pp.bias_scale = 1.4426950408889634f;
  const int grid = pp.num_tiles < sm_count() ? pp.num_tiles : sm_count();
  if (f32)
    triatt_proj_kernel<true><<<grid, triatt_proj::THREADS, triatt_proj::SMEM_BYTES, stream>>>(tmW, tmQKG, tmVT, tmWB, pp);
  else
    triatt_proj_kernel<false><<<grid, triatt_proj::THREADS, triatt_proj::SMEM_BYTES, stream>>>(tmW, tmQKG, tmVT, tmWB, pp);
  B200_AFTER_LAUNCH();
  {
    FlashLaunch a;
    a.qk = qkg;
    a.qk_width = 384;
    a.qk_b_stride = int64_t(pos) * 384;
    a.vT = vT;
    a.v_pitch = pl.Nk;
    a.bias = ext_bias ? ext_bias : static_cast<const void*>(tb);
    a.bias_pitch = ext_bias ? ext_bias_pitch : pl.Nk;
    a.bias_groups = 1;
    FlashParams& p = a.p;
    p.mask = mask;
    p.mask_div = 1;
    // line l attends over keys k with mask[l][k] (starting node) or mask[k][l] (ending node)
    p.mask_row_stride = ending ? 1 : n_cols;
    p.mask_key_stride = ending ? n_cols : 1;
    p.bias_div = lines;
    p.gate = qkg;
    p.gate_activated = 1;  // the projection kernel stores sigmoid(g)
    p.gate_b_stride = int64_t(pos) * 384;
    p.gate_pitch = 384;
    p.gate_col0 = 256;
    p.out = og;
    p.out_b_stride = int64_t(pos) * kD;
    p.out_pitch = kD;
    p.out_col0 = 0;
    p.dh_out = 32;
    p.N = pos;
    p.H = 4;
    p.Bt = lines;
    p.q_col0 = 0;
    p.k_col0 = 128;
    p.v_row0 = 0;
    if (int e = launch_flash(a, 32, stream)) return e;
  }
  {
    BmmLaunch a{og, w->w_o, out, 1, lines * pos, kD, kD, kD, kD, kD, 0, 0, 0};
    a.out_f32 = f32;
    a.residual = add_residual ? z : nullptr;
    a.remap_n = ending ? pos : 0;
    a.remap_m = ending ? lines : 0;
    if (int e = launch_bmm(a, stream)) return e;
  }
  return B200_OK;
}

static bool triatt_weights_ok(const b200_triatt_weights* w) {
  return w && w->w_qkgv && w->g_bias && w->w_b && w->w_o && w->ln_w && w->ln_b;
}

size_t b200_triatt_workspace_bytes(int N) {
  if (N <= 0) return 0;
  TriAttPlan pl;
  triatt_plan(N, N, true, &pl);
  return pl.total;
}

size_t b200_triatt_slab_workspace_bytes(int n_rows, int n_cols, int ending) {
  if (n_rows <= 0 || n_cols <= 0) return 0;
  TriAttPlan pl;
  triatt_plan(ending ? n_cols : n_rows, ending ? n_rows : n_cols, false, &pl);
  return pl.total;
}

int b200_triatt_fwd(const void* z, const uint8_t* mask, void* out, const b200_triatt_weights* w, int B, int N,
                    int ending, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                    b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(z && mask && out, "z/mask/out is NULL");
  B200_CHECK_ARG(triatt_weights_ok(w), "a weight pointer is NULL");
  B200_CHECK_ARG(B > 0 && N > 0, "B=%d, N=%d must be positive", B, N);
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown z_dtype %d", z_dtype);
  B200_CHECK_ARG(aligned(z, 32) && aligned(out, 32), "z/out must be 32-byte aligned");
  const bool f32 = z_dtype == B200_DTYPE_F32;
  const size_t esz = f32 ? 4 : 2;
  for (int bi = 0; bi < B; ++bi) {
    const size_t off = size_t(bi) * N * N * kD * esz;
    if (int e = triatt_slab(static_cast<const uint8_t*>(z) + off, mask + size_t(bi) * N * N, nullptr, 0,
                            static_cast<uint8_t*>(out) + off, w, N, N, ending != 0, add_residual != 0, f32, workspace,
                            workspace_bytes, static_cast<cudaStream_t>(stream_)))
      return e;
  }
  return B200_OK;
}

int b200_triatt_slab_fwd(const void* z, const uint8_t* mask, const void* bias, int64_t bias_pitch, void* out,
                         const b200_triatt_weights* w, int n_rows, int n_cols, int ending, int add_residual, int z_dtype,
                         void* workspace, size_t workspace_bytes, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(z && mask && bias && out, "z/mask/bias/out is NULL");
  B200_CHECK_ARG(triatt_weights_ok(w), "a weight pointer is NULL");
  B200_CHECK_ARG(n_rows > 0 && n_cols > 0, "n_rows=%d, n_cols=%d must be positive", n_rows, n_cols);
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown z_dtype %d", z_dtype);
  B200_CHECK_ARG(aligned(z, 32) && aligned(out, 32) && aligned(bias, 16), "z/out must be 32-byte aligned, bias 16-byte");
  const int pos = ending ? n_rows : n_cols;
  B200_CHECK_ARG(bias_pitch % 8 == 0 && bias_pitch >= pos, "bias pitch must be a multiple of 8 and >= %d", pos);
  return triatt_slab(z, mask, bias, bias_pitch, out, w, n_rows, n_cols, ending != 0, add_residual != 0,
                     z_dtype == B200_DTYPE_F32, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------ single-track helpers
static int grid_for(int64_t work_items, int per_block) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  const int64_t cap = int64_t(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return int(blocks);
}

int b200_rows_to_bf16(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, int x_dtype,
                      int normalize, int silu, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && y, "x/y is NULL");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= 1024, "cols=%d must be a multiple of 8, <= 1024", cols);
  B200_CHECK_ARG((x_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x, 32) && aligned(y, 16), "x must be 32-byte aligned, y 16-byte aligned");
  if (rows == 0) return B200_OK;
  return launch_rows_to_bf16(x, x_dtype == B200_DTYPE_F32, static_cast<__nv_bfloat16*>(y), w, b, rows, cols,
                             normalize != 0, static_cast<cudaStream_t>(stream), silu != 0);
}

int b200_rows2_to_bf16(const void* x1, int cols1, const void* x2, int cols2, void* y, const float* w, const float* b,
                       int64_t rows, int x_dtype, int normalize, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x1 && x2 && y, "x1/x2/y is NULL");
  B200_CHECK_ARG(rows >= 0 && cols1 > 0 && cols2 > 0 && cols1 % 8 == 0 && cols2 % 8 == 0 && cols1 + cols2 <= 1024,
                 "cols1=%d and cols2=%d must be positive multiples of 8 with a sum <= 1024", cols1, cols2);
  B200_CHECK_ARG((x_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x1, 32) && aligned(x2, 32) && aligned(y, 16), "x1/x2 must be 32-byte aligned, y 16-byte aligned");
  if (rows == 0) return B200_OK;
  return launch_rows_to_bf16(x1, x_dtype == B200_DTYPE_F32, static_cast<__nv_bfloat16*>(y), w, b, rows, cols1 + cols2,
                             normalize != 0, static_cast<cudaStream_t>(stream), false, x2, cols1);
}

int b200_window_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const float* w_z, float* bias,
                         int64_t windows, int W, int Hk, int c_z, int heads, int z_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(z && ln_w && w_z && bias, "z/ln_w/w_z/bias is NULL");
  B200_CHECK_ARG(windows >= 0 && W > 0 && Hk > 0, "need windows >= 0 and W, Hk > 0");
  B200_CHECK_ARG(c_z > 0 && c_z % 4 == 0 && c_z <= 128, "c_z=%d must be a multiple of 4, at most 128", c_z);
  B200_CHECK_ARG(aligned(z, 16) && aligned(bias, 4), "z must be 16-byte aligned");
  B200_CHECK_ARG(heads > 0 && heads <= kWindowMaxHeads, "heads=%d must be in 1..%d", heads, kWindowMaxHeads);
  B200_CHECK_ARG((z_dtype | 1) == 1, "unknown dtype");
  if (windows == 0) return B200_OK;
  WindowBiasParams p{z, ln_w, ln_b, w_z, bias, windows * W * Hk, W * Hk, c_z, heads, 1e-5f};
  int lpr = 1;
  while (lpr * 4 < c_z) lpr *= 2;  // lanes per pair: four channels each
  const int grid = grid_for(p.pairs * lpr, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (z_dtype == B200_DTYPE_F32) window_bias_kernel<true><<<grid, 256, 0, st>>>(p, lpr);
  else window_bias_kernel<false><<<grid, 256, 0, st>>>(p, lpr);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_window_attention_fwd(const void* qkv, const void* gate, const float* bias, const uint8_t* mask, void* out, int B,
                              int M, int NW, int W, int Hk, int heads, int head_dim, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(qkv && gate && bias && mask && out, "qkv/gate/bias/mask/out is NULL");
  B200_CHECK_ARG(B > 0 && M > 0 && NW > 0 && W > 0 && Hk >= W && Hk % 8 == 0 && (Hk - W) % 2 == 0,
                 "need B, M, NW, W > 0 and Hk >= W, a multiple of 8, with Hk - W even (W=%d, Hk=%d)", W, Hk);
  B200_CHECK_ARG(heads > 0 && heads * W <= 256, "heads * W = %d exceeds the 256 threads of a window's CTA", heads * W);
  B200_CHECK_ARG(head_dim == 16 || head_dim == 32 || head_dim == 64, "head_dim=%d must be 16, 32 or 64", head_dim);
  B200_CHECK_ARG(2ll * Hk * heads * head_dim * 2 + Hk + 16 <= 227 * 1024, "the key window does not fit in shared memory");
  B200_CHECK_ARG((int64_t)B * M * NW < (int64_t(1) << 31), "too many windows");
  B200_CHECK_ARG(aligned(qkv, 16) && aligned(gate, 16) && aligned(out, 16) && aligned(bias, 16),
                 "qkv/gate/out/bias must be 16-byte aligned");
  WindowAttnParams p{static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(gate), bias, mask,
                     static_cast<__nv_bfloat16*>(out), NW, W, Hk, heads, M, 1.0f / sqrtf(float(head_dim))};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 16) return launch_window_attention<16>(p, B * M, st);
  if (head_dim == 32) return launch_window_attention<32>(p, B * M, st);
  return launch_window_attention<64>(p, B * M, st);
}

int b200_pair_outer_sum(const float* a, const float* c, const float* extra, float* z, int n_i, int n_j, int cols,
                        b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(a && c && z, "a/c/z is NULL");
  B200_CHECK_ARG(n_i >= 0 && n_j >= 0 && cols > 0 && cols % 8 == 0, "cols=%d must be a positive multiple of 8", cols);
  B200_CHECK_ARG(aligned(a, 32) && aligned(c, 32) && aligned(z, 32) && (!extra || aligned(extra, 32)),
                 "a/c/extra/z must be 32-byte aligned");
  if (n_i == 0 || n_j == 0) return B200_OK;
  pair_outer_sum_kernel<<<grid_for((int64_t)n_i * n_j * (cols / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, c, extra, z, n_i, n_j, cols);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_add_rows(const float* x, const void* y, float* out, int64_t rows, int64_t period, int cols, int y_dtype,
                  b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && y && out, "x/y/out is NULL");
  B200_CHECK_ARG(rows >= 0 && period > 0 && cols > 0 && cols % 8 == 0, "need period > 0 and cols a positive multiple of 8");
  B200_CHECK_ARG((y_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x, 32) && aligned(y, 32) && aligned(out, 32), "x/y/out must be 32-byte aligned");
  if (rows == 0) return B200_OK;
  const int grid = grid_for(rows * (cols / 8), 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (y_dtype == B200_DTYPE_F32) add_rows_kernel<true><<<grid, 256, 0, st>>>(x, y, out, rows, period, cols);
  else add_rows_kernel<false><<<grid, 256, 0, st>>>(x, y, out, rows, period, cols);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_linear_bf16(const void* x, const void* w, const float* bias, const void* residual, void* out, int64_t rows,
                     int in_features, int out_features, int out_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && w && out, "x/w/out is NULL");
  B200_CHECK_ARG(rows > 0 && rows < (int64_t(1) << 31), "rows out of range");
  B200_CHECK_ARG(in_features > 0 && in_features % 8 == 0 && out_features > 0 && out_features % 8 == 0,
                 "in_features=%d and out_features=%d must be positive multiples of 8", in_features, out_features);
  B200_CHECK_ARG((out_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x, 16) && aligned(w, 16) && aligned(out, 32) && (!residual || aligned(residual, 32)),
                 "x/w must be 16-byte aligned, out/residual 32-byte aligned");
  BmmLaunch a{x, w, out, 1, int(rows), out_features, in_features, in_features, in_features, out_features, 0, 0, 0};
  a.bias = bias;
  a.residual = residual;
  a.out_f32 = out_dtype == B200_DTYPE_F32;
  return launch_bmm(a, static_cast<cudaStream_t>(stream));
}

int b200_swiglu_fwd(const void* h12, void* h, int64_t rows, int hidden, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(h12 && h, "h12/h is NULL");
  B200_CHECK_ARG(rows >= 0 && hidden > 0 && hidden % 8 == 0, "hidden=%d must be a positive multiple of 8", hidden);
  B200_CHECK_ARG(aligned(h12, 16) && aligned(h, 16), "h12/h must be 16-byte aligned");
  if (rows == 0) return B200_OK;
  swiglu_rows_kernel<<<grid_for(rows * (hidden / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h12), static_cast<__nv_bfloat16*>(h), rows, hidden);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_adaln_fwd(const void* x, const float* cond, int cond_width, int alpha_col, int beta_col, float lns, void* y,
                   int64_t rows, int cols, int x_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && cond && y, "x/cond/y is NULL");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= 1024, "cols=%d must be a multiple of 8, <= 1024", cols);
  B200_CHECK_ARG(cond_width % 8 == 0 && alpha_col % 8 == 0 && beta_col % 8 == 0 && alpha_col + cols <= cond_width &&
                     beta_col + cols <= cond_width, "bad conditioning layout");
  B200_CHECK_ARG((x_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x, 32) && aligned(cond, 32) && aligned(y, 16), "x/cond must be 32-byte aligned, y 16-byte");
  if (rows == 0) return B200_OK;
  const int grid = grid_for(rows, 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dtype == B200_DTYPE_F32)
    adaln_rows_kernel<true><<<grid, 256, 0, st>>>(x, cond, cond_width, alpha_col, beta_col, lns,
                                                  static_cast<__nv_bfloat16*>(y), rows, cols, 1e-5f);
  else
    adaln_rows_kernel<false><<<grid, 256, 0, st>>>(x, cond, cond_width, alpha_col, beta_col, lns,
                                                   static_cast<__nv_bfloat16*>(y), rows, cols, 1e-5f);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_gated_residual_fwd(void* x, const void* h, const float* cond, int cond_width, int gamma_col, int64_t rows,
                            int cols, int x_dtype, int h_dtype, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && h && cond, "x/h/cond is NULL");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0, "cols=%d must be a positive multiple of 8", cols);
  B200_CHECK_ARG(cond_width % 8 == 0 && gamma_col % 8 == 0 && gamma_col + cols <= cond_width, "bad conditioning layout");
  B200_CHECK_ARG((x_dtype | 1) == 1 && (h_dtype | 1) == 1, "unknown dtype");
  B200_CHECK_ARG(aligned(x, 32) && aligned(h, 32) && aligned(cond, 32), "x/h/cond must be 32-byte aligned");
  if (rows == 0) return B200_OK;
  const int grid = grid_for(rows * (cols / 8), 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool xf = x_dtype == B200_DTYPE_F32, hf = h_dtype == B200_DTYPE_F32;
  if (xf && hf) gated_residual_rows_kernel<true, true><<<grid, 256, 0, st>>>(x, h, cond, cond_width, gamma_col, rows, cols);
  else if (xf) gated_residual_rows_kernel<true, false><<<grid, 256, 0, st>>>(x, h, cond, cond_width, gamma_col, rows, cols);
  else if (hf) gated_residual_rows_kernel<false, true><<<grid, 256, 0, st>>>(x, h, cond, cond_width, gamma_col, rows, cols);
  else gated_residual_rows_kernel<false, false><<<grid, 256, 0, st>>>(x, h, cond, cond_width, gamma_col, rows, cols);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_masked_softmax_rows(const void* logits, const uint8_t* mask, void* out, int H, int n_rows, int n, int pitch,
                             b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(logits && mask && out, "logits/mask/out is NULL");
  B200_CHECK_ARG(H > 0 && n > 0 && n_rows > 0 && pitch >= n && pitch % 8 == 0,
                 "need H, n_rows, n > 0 and a pitch >= n that is a multiple of 8");
  B200_CHECK_ARG(aligned(logits, 16) && aligned(out, 16), "logits/out must be 16-byte aligned");
  masked_softmax_rows_kernel<<<grid_for((int64_t)H * n_rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), mask, static_cast<__nv_bfloat16*>(out), H, n_rows, n, pitch);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_pwa_gate(const void* o, const void* g, void* og, int S, int n, int H, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(o && g && og, "o/g/og is NULL");
  B200_CHECK_ARG(S > 0 && n > 0 && H > 0, "S, n, H must be positive");
  B200_CHECK_ARG(aligned(o, 16) && aligned(g, 16) && aligned(og, 16), "o/g/og must be 16-byte aligned");
  pwa_gate_kernel<<<grid_for((int64_t)S * n * H * 4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(og), S, n, H);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_split_rows(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, float eps,
                    int normalize, int order, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(x && y, "x/y is NULL");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0, "cols=%d must be a positive multiple of 8", cols);
  B200_CHECK_ARG(!normalize || cols <= 1024, "LayerNorm rows hold at most 1024 channels");
  B200_CHECK_ARG(order == 0 || order == 1, "order must be 0 (hi|hi|lo) or 1 (hi|lo|hi)");
  B200_CHECK_ARG(aligned(x, 32) && aligned(y, 16), "x must be 32-byte aligned, y 16-byte aligned");
  if (rows == 0) return B200_OK;
  split_rows_kernel<<<grid_for(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y), w, b, rows, cols, eps, normalize, order);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_gate_rows_f32(const float* a, int64_t a_pitch, const float* b, int64_t b_pitch, const uint8_t* rowmask,
                       float* out, int64_t rows, int cols, int mode, b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(a && b && out, "a/b/out is NULL");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 4 == 0 && a_pitch % 4 == 0 && b_pitch % 4 == 0,
                 "cols and the pitches must be multiples of 4");
  B200_CHECK_ARG(mode >= 0 && mode <= 2, "mode must be 0 (a * sigmoid(b)), 1 (silu(a) * b) or 2 (a)");
  B200_CHECK_ARG(aligned(a, 16) && aligned(b, 16) && aligned(out, 16), "a/b/out must be 16-byte aligned");
  if (rows == 0) return B200_OK;
  gate_rows_f32_kernel<<<grid_for(rows * (cols / 4), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, a_pitch, b, b_pitch, rowmask, out, rows, cols, mode);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

int b200_softmax_bias_f32(float* s, const float* bias, const uint8_t* keymask, int64_t groups, int n, int H, int bias_div,
                          b200_stream_t stream) {
  if (int e = b200_check_device()) return e;
  B200_CHECK_ARG(s && keymask, "s/keymask is NULL");
  B200_CHECK_ARG(groups > 0 && n > 0 && H > 0 && bias_div > 0 && groups % ((int64_t)H * bias_div) == 0,
                 "groups must be a multiple of H * bias_div");
  softmax_bias_f32_kernel<<<grid_for(groups * n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      s, bias, keymask, groups, n, H, bias_div, H * bias_div);
  B200_AFTER_LAUNCH();
  return B200_OK;
}

}  // extern "C"
