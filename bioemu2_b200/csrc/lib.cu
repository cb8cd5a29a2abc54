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

namespace b200 {

template <class Kernel>
static int set_smem(Kernel k, uint32_t bytes) {
  B200_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
  return 0;
}

static int launch_bmm(const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, int64_t sa, int64_t sb, int64_t sc, float scale,
                      cudaStream_t stream) {
  const int BN = (N % 256 == 0 || N > 1024) ? 256 : 128;
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[3] = {uint64_t(K), uint64_t(M), uint64_t(batch)};
    const uint64_t str[2] = {uint64_t(lda) * 2, uint64_t(sa) * 2};
    const uint32_t box[3] = {64, 128, 1};
    if (int e = make_tmap_bf16(&tmA, A, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(K), uint64_t(N), uint64_t(batch)};
    const uint64_t str[2] = {uint64_t(ldb) * 2, uint64_t(sb) * 2};
    const uint32_t box[3] = {64, uint32_t(BN), 1};
    if (int e = make_tmap_bf16(&tmB, B, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  BmmParams p;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.c_batch_stride = sc;
  p.ldc = int(ldc);
  p.m_valid = M;
  p.n_valid = N;
  p.tiles_m = (M + 127) / 128;
  p.tiles_n = (N + BN - 1) / BN;
  p.batch = batch;
  p.k_blocks = (K + 63) / 64;
  p.scale = scale;
  const int total = p.tiles_m * p.tiles_n * batch;
  const int grid = total < sm_count() ? total : sm_count();
  if (BN == 256) {
    if (int e = set_smem(bmm_nt_kernel<256>, BmmCfg<256>::SMEM_BYTES)) return e;
    bmm_nt_kernel<256><<<grid, 192, BmmCfg<256>::SMEM_BYTES, stream>>>(tmA, tmB, p);
  } else {
    if (int e = set_smem(bmm_nt_kernel<128>, BmmCfg<128>::SMEM_BYTES)) return e;
    bmm_nt_kernel<128><<<grid, 192, BmmCfg<128>::SMEM_BYTES, stream>>>(tmA, tmB, p);
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_version(void) { return 100; }

const char* b200_last_error(void) { return g_last_error; }

int b200_check_device(void) {
  static thread_local int cached_dev = -1;
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev == cached_dev) return B200_OK;
  int major = 0;
  B200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return fail(B200_ERR_UNSUPPORTED_DEVICE, "device %d has compute capability %d.x; this library is sm_100a only",
                dev, major);
  cached_dev = dev;
  return B200_OK;
}

int b200_device_status(int* status) {
  B200_CHECK_ARG(status != nullptr, "status is NULL");
  B200_CUDA(cudaDeviceSynchronize());
  int v = 0;
  B200_CUDA(cudaMemcpyFromSymbol(&v, g_dev_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    B200_CUDA(cudaMemcpyToSymbol(g_dev_status, &zero, sizeof(int)));
  }
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
  layernorm_rows_kernel<<<int(blocks), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), w, b, rows, cols, eps);
  B200_CUDA(cudaGetLastError());
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
  B200_CHECK_ARG(lda >= K && ldb >= K && ldc >= N, "row pitch smaller than the row");
  B200_CHECK_ARG(aligned(A, 16) && aligned(B, 16) && aligned(C, 16), "A/B/C must be 16-byte aligned");
  return launch_bmm(A, B, C, batch, M, N, K, lda, ldb, ldc, sa, sb, sc, scale, static_cast<cudaStream_t>(stream));
}

static inline int padded_n(int N) { return (N + 127) / 128 * 128; }

size_t b200_trimul_workspace_bytes(int N) {
  if (N <= 0) return 0;
  const size_t Np = size_t(padded_n(N));
  return 3 * size_t(kD) * Np * Np * sizeof(__nv_bfloat16);  // a, b, t
}

int b200_trimul_fwd(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                    int incoming, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                    b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(z && mask && out && w, "z/mask/out/w is NULL");
  B200_CHECK_ARG(w->w_in && w->w_out && w->ln_in_w && w->ln_in_b && w->ln_out_w && w->ln_out_b,
                 "a weight pointer is NULL");
  B200_CHECK_ARG(B > 0 && N > 0, "B=%d, N=%d must be positive", B, N);
  B200_CHECK_ARG(z_dtype == B200_DTYPE_BF16 || z_dtype == B200_DTYPE_F32, "unknown z_dtype %d", z_dtype);
  B200_CHECK_ARG(aligned(z, 32) && aligned(out, 32) && aligned(w->w_in, 16) && aligned(w->w_out, 16),
                 "z/out must be 32-byte aligned, weights 16-byte aligned");
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

  CUtensorMap tmWin, tmWout, tmT;
  {
    const uint64_t dims[2] = {128, 512};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmWin, w->w_in, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[2] = {128, 256};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (int e = make_tmap_bf16(&tmWout, w->w_out, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  }
  {
    const uint64_t dims[3] = {uint64_t(Np), uint64_t(Np), uint64_t(kD)};
    const uint64_t str[2] = {uint64_t(Np) * 2, uint64_t(Np) * Np * 2};
    const uint32_t box[3] = {128, 1, 128};
    if (int e = make_tmap_bf16(&tmT, t_buf, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
  }
  if (int e = set_smem(trimul_in_kernel<true>, trimul_in::SMEM_BYTES)) return e;
  if (int e = set_smem(trimul_in_kernel<false>, trimul_in::SMEM_BYTES)) return e;
  if (int e = set_smem(trimul_out_kernel<true>, trimul_out::SMEM_BYTES)) return e;
  if (int e = set_smem(trimul_out_kernel<false>, trimul_out::SMEM_BYTES)) return e;

  const int num_tiles = N * (Np / 128);
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  for (int bi = 0; bi < B; ++bi) {
    const uint8_t* zb = static_cast<const uint8_t*>(z) + size_t(bi) * N * N * kD * esz;
    uint8_t* ob = static_cast<uint8_t*>(out) + size_t(bi) * N * N * kD * esz;
    TriMulInParams pi;
    pi.z = zb;
    pi.mask = mask + size_t(bi) * N * N;
    pi.ln_w = w->ln_in_w;
    pi.ln_b = w->ln_in_b;
    pi.a_out = a_buf;
    pi.b_out = b_buf;
    pi.N = N;
    pi.Np = Np;
    pi.incoming = incoming ? 1 : 0;
    pi.num_tiles = num_tiles;
    pi.eps = 1e-5f;
    if (f32)
      trimul_in_kernel<true><<<grid, trimul_in::THREADS, trimul_in::SMEM_BYTES, stream>>>(tmWin, pi);
    else
      trimul_in_kernel<false><<<grid, trimul_in::THREADS, trimul_in::SMEM_BYTES, stream>>>(tmWin, pi);
    B200_CUDA(cudaGetLastError());

    if (int e = launch_bmm(a_buf, b_buf, t_buf, kD, Np, Np, Np, Np, Np, Np, int64_t(Np) * Np, int64_t(Np) * Np,
                           int64_t(Np) * Np, 1.0f, stream))
      return e;

    TriMulOutParams po;
    po.z = zb;
    po.out = ob;
    po.ln_in_w = w->ln_in_w;
    po.ln_in_b = w->ln_in_b;
    po.ln_out_w = w->ln_out_w;
    po.ln_out_b = w->ln_out_b;
    po.N = N;
    po.Np = Np;
    po.num_tiles = num_tiles;
    po.add_residual = add_residual ? 1 : 0;
    po.eps = 1e-5f;
    if (f32)
      trimul_out_kernel<true><<<grid, trimul_out::THREADS, trimul_out::SMEM_BYTES, stream>>>(tmWout, tmT, po);
    else
      trimul_out_kernel<false><<<grid, trimul_out::THREADS, trimul_out::SMEM_BYTES, stream>>>(tmWout, tmT, po);
    B200_CUDA(cudaGetLastError());
  }
  return B200_OK;
}

int b200_transition_fwd(const void* x, void* out, const void* w13, const void* w3, const float* ln_w,
                        const float* ln_b, int64_t rows, int use_norm, int add_residual, int x_dtype,
                        b200_stream_t stream_) {
  if (int e = b200_check_device()) return e;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_CHECK_ARG(x && out && w13 && w3, "x/out/w13/w3 is NULL");
  B200_CHECK_ARG(!use_norm || (ln_w && ln_b), "use_norm needs ln_w and ln_b");
  B200_CHECK_ARG(rows >= 0 && rows < (int64_t(1) << 31) * 128, "rows out of range");
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
    transition_kernel<true><<<grid, transition::THREADS, transition::SMEM_BYTES, stream>>>(tmW1, tmW3, p);
  else
    transition_kernel<false><<<grid, transition::THREADS, transition::SMEM_BYTES, stream>>>(tmW1, tmW3, p);
  B200_CUDA(cudaGetLastError());
  return B200_OK;
}

}  // extern "C"
