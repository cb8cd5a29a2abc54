/*
 * b200pair -- C ABI of the B200 (sm_100a) kernels for the pair-representation hot path.
 *
 * The reference project is pure PyTorch: its seam for this path is the nn.Module contract of the ops
 * (there is no FFI to mirror), so each entry point below names the reference module method whose
 * arithmetic it replaces.  Conventions shared by all entry points:
 *
 *   - every pointer is a DEVICE pointer borrowed for the duration of the call, unless it says "host";
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); nothing synchronises;
 *   - nothing is allocated: scratch comes from the caller (`*_workspace_bytes` says how much);
 *   - activations are bf16, LayerNorm parameters fp32, projection weights bf16 in the packed layouts
 *     described per function (the Python modules in bioemu2_b200/ build them from the reference's
 *     state_dict tensors);
 *   - the return value is a status code (B200_OK == 0); b200_last_error() gives the message of the
 *     calling thread's last failure.  No exception crosses the boundary.
 *   - kernels bound every wait; if one runs out the kernel finishes with wrong data, writes a status word, and
 *     every later compute entry point on that device returns B200_ERR_DEVICE_WAIT until b200_device_status()
 *     has read and cleared it (b200_peek_status() reads it without synchronising).  Kernels that were already
 *     enqueued behind the failing one still run, and finish early with invalid results.
 */
#ifndef B200PAIR_H_
#define B200PAIR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_ERR_INVALID_ARGUMENT 1
#define B200_ERR_CUDA 2
#define B200_ERR_UNSUPPORTED_DEVICE 3
#define B200_ERR_WORKSPACE 4
#define B200_ERR_DEVICE_WAIT 5

typedef void* b200_stream_t; /* cudaStream_t */

/* Element type of the pair tensor ("z stream") an entry point reads and writes.  The reference keeps the
 * pair tensor in fp32 even under bf16 autocast (the residual adds promote), so fp32 is the trunk's type;
 * bf16 serves callers that hold a bf16 pair tensor.  Arithmetic is the same for both: bf16 tensor-core
 * operands, fp32 accumulation, fp32 LayerNorm / gating / residual. */
#define B200_DTYPE_BF16 0
#define B200_DTYPE_F32 1

/* Library version (major*100 + minor). */
int b200_version(void);

/* Message of the calling thread's most recent failure ("" if none). */
const char* b200_last_error(void);

/* Checks that the current device is compute capability 10.x and that no earlier kernel on it gave up a bounded
 * wait (B200_ERR_DEVICE_WAIT otherwise).  Every compute entry point calls it first.  The first call on a device
 * sets up 64 bytes of pinned host memory through which kernels report such a failure; make that first call
 * outside any stream capture. */
int b200_check_device(void);

/* Synchronises the device, then reads and clears the device status word into *status (host pointer).
 * 0 = every kernel wait completed; otherwise low byte 1 = a bounded wait ran out, bits 8.. = its site. */
int b200_device_status(int* status);

/* The same word as far as kernels that have FINISHED wrote it, read from host memory: no synchronisation, no
 * CUDA call on the fast path, nothing cleared.  For polling between launches (before a device-to-host copy, before
 * a collective, at the end of a forward). */
int b200_peek_status(int* status);

/* Number of kernels this library has launched since it was loaded (all threads, all devices). */
unsigned long long b200_launch_count(void);

/* ---------------------------------------------------------------------------------------------------
 * Row LayerNorm: y[r,:] = (x[r,:] - mean) * rsqrt(var + eps) * w + b over `cols` (multiple of 8, <= 1024).
 * Replaces torch.nn.LayerNorm as used by norm_in / norm_s / norm_z
 * (src/bioemu2/biomoa/ops/triangle_multiplication.py:71, attention_pair_bias.py:85,90).
 * w or b may be NULL (no scale / no shift).
 * ------------------------------------------------------------------------------------------------- */
int b200_layernorm_fwd(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, float eps,
                       b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Batched C[b] = scale * A[b] * B[b]^T, bf16 in / bf16 out, fp32 accumulation on the tensor cores.
 * A: [batch][M][K] (row pitch lda elements), B: [batch][N][K] (pitch ldb), C: [batch][M][N] (pitch ldc).
 * Pitches and batch strides are in elements and must be multiples of 8; N multiple of 8.
 * Replaces the per-channel einsum of TriangleMultiplicationFull.forward
 * (src/bioemu2/biomoa/ops/triangle_multiplication.py:94-98) and the MSA-depth contraction of
 * OuterProductMeanVanilla.forward (src/bioemu2/biomoa/ops/outer_product_mean.py:71).
 * ------------------------------------------------------------------------------------------------- */
int b200_bmm_nt_bf16(const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda,
                     int64_t ldb, int64_t ldc, int64_t a_batch_stride, int64_t b_batch_stride,
                     int64_t c_batch_stride, float scale, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Triangle multiplication, TriangleMultiplicationFull.forward
 * (src/bioemu2/biomoa/ops/triangle_multiplication.py:86-99; weights :62-76), c_z = 128.
 *
 *   w_in   bf16 [512][128]: rows 0..127 = p_in.weight[0:128], 128..255 = g_in.weight[0:128],
 *                           256..383 = p_in.weight[128:256], 384..511 = g_in.weight[128:256]
 *   w_out  bf16 [256][128]: rows 0..127 = p_out.weight, 128..255 = g_out.weight
 *   ln_*   fp32 [128]
 *
 * z, out: [B][N][N][128] of `z_dtype`; mask: uint8 [B][N][N] (non-zero = valid).  `out` may alias `z`.
 * incoming: 0 = outgoing ("bikd,bjkd->bijd"), 1 = incoming ("bkid,bkjd->bijd").
 * add_residual: 0 returns the update as the reference op does; 1 returns z + update, which is what
 * PairMixerLayer.forward does with it (src/bioemu2/biomoa/modules/pairmixer.py:447-452).
 * Workspace: b200_trimul_workspace_bytes(N) bytes, 1024-byte aligned.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
  const void* w_in;
  const void* w_out;
  const float* ln_in_w;
  const float* ln_in_b;
  const float* ln_out_w;
  const float* ln_out_b;
} b200_trimul_weights;

size_t b200_trimul_workspace_bytes(int N);

int b200_trimul_fwd(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                    int incoming, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                    b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Triangle multiplication in stages, for callers that shard the pair tensor (the 2D context-parallel form,
 * src/bioemu2/context_parallel/ops/triangle_multiplication.py:45-182 and ops/triangular_mult_impl.py:113-385):
 * the projection and the output stage run on a rectangular slab z[n_rows][n_cols][128] (row pitch
 * z_row_stride elements), the contraction is b200_bmm_nt on whatever the caller has gathered in between.
 *
 * b200_trimul_project  a, b = halves of mask * p_in(LN_in(z)) * sigmoid(g_in(LN_in(z))), written channel-major
 *                      [128][lines][pos_pitch] bf16 with (line, pos) = (row, column) for incoming = 0 and
 *                      (column, row) for incoming = 1; positions >= n_pos are written as zero up to pos_pitch
 *                      (a multiple of 128), so the buffers can be used as zero-padded K-major GEMM operands.
 * b200_trimul_output   out = p_out(LN_out(t)) * sigmoid(g_out(LN_in(z))) [+ z] on the slab, with t bf16
 *                      [128][lines][pos_pitch] indexed (row, column), or (column, row) when transposed_t = 1.
 * b200_bmm_nt          b200_bmm_nt_bf16 with a selectable output type (fp32 for partial sums that are reduced
 *                      across GPUs afterwards).
 * ------------------------------------------------------------------------------------------------- */
int b200_trimul_project(const void* z, const uint8_t* mask, void* a_out, void* b_out, const b200_trimul_weights* w,
                        int n_rows, int n_cols, int64_t z_row_stride, int64_t mask_row_stride, int incoming,
                        int pos_pitch, int z_dtype, b200_stream_t stream);
int b200_trimul_output(const void* t, const void* z, void* out, const b200_trimul_weights* w, int n_rows, int n_cols,
                       int64_t z_row_stride, int transposed_t, int pos_pitch, int add_residual, int z_dtype,
                       b200_stream_t stream);
int b200_bmm_nt(const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda, int64_t ldb,
                int64_t ldc, int64_t a_batch_stride, int64_t b_batch_stride, int64_t c_batch_stride, float scale,
                int out_dtype, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Triangle multiplication without a caller workspace and without any allocation.
 * (No counterpart in the reference: it exists for callers of this library that must not allocate device
 * memory -- a serving loop whose memory is fully handed to another framework's pool, a latency-critical
 * thread where cudaMalloc's implicit device synchronisation is not acceptable, or an embedding host that
 * simply has no allocator to lend a workspace from.)
 *
 * Same arguments and results as b200_trimul_fwd, minus the workspace: the scratch is a fixed array inside the
 * library image, 48 MiB per GPU that loads the library, held until the process exits.  Limit: N <= 256;
 * larger N is rejected with B200_ERR_INVALID_ARGUMENT.  The call makes no cudaMalloc/cudaFree and calls no
 * allocating library routine.  The first call on each device resolves the array's device address
 * (cudaGetSymbolAddress with that device current); make that first call outside any stream capture.
 * All calls on a device share the one array: calls that may overlap on the GPU (different streams) race and
 * must be serialised by the caller.  Nothing in the array needs to start at zero, so it is not cleared between
 * calls: the planes are padded to a multiple of 128 rows and columns, the padding may hold what an earlier call
 * left there (any bit pattern), and it is read only into padded rows and columns of the intermediate products,
 * whose results are never stored to the output.
 * ------------------------------------------------------------------------------------------------- */
int b200_trimul_fwd_static(const void* z, const uint8_t* mask, void* out, const b200_trimul_weights* w, int B, int N,
                           int incoming, int add_residual, int z_dtype, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Pair transition, Transition.forward (src/bioemu2/biomoa/ops/transition.py:52-76) for dim 128, hidden 512:
 * out = fc3(silu(fc1(h)) * fc2(h)) [+ x], h = LayerNorm(x) when use_norm else x.
 *
 *   w13  bf16 [1024][128]: for hidden chunk c = 0..7, rows c*128 + 0..63 = fc1.weight[c*64 + 0..63],
 *                          rows c*128 + 64..127 = fc2.weight[c*64 + 0..63]
 *   w3   bf16 [128][512] = fc3.weight
 *
 * x, out: [rows][128] of `x_dtype`; `out` may alias `x`.
 * ------------------------------------------------------------------------------------------------- */
int b200_transition_fwd(const void* x, void* out, const void* w13, const void* w3, const float* ln_w,
                        const float* ln_b, int64_t rows, int use_norm, int add_residual, int x_dtype,
                        b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Outer product mean, OuterProductMeanVanilla.forward (src/bioemu2/biomoa/ops/outer_product_mean.py:45-75)
 * for c_in = 64, c_hidden = 32, c_out = 128:
 *   m' = mask * proj_ab(LN(m));  a, b = halves of m';  out[i,j,:] = proj_o(vec(sum_s a[s,i,:] (x) b[s,j,:]) / n) + bias
 * with n = number of MSA rows holding at least one valid token (clamped to >= 1) for a [B,S,N] mask
 * (mask_ndim 3) and n = 1 for a [B,N] mask (mask_ndim 2, B must be 1, as in the reference where only that
 * shape broadcasts).  The S-contraction accumulates in fp32 on the tensor cores and is rounded to bf16
 * once, before proj_o, as the reference's `z.to(m)` does under autocast.
 *
 *   w_ab  bf16 [64][64]    = proj_ab.weight        ln_w, ln_b  fp32 [64]
 *   w_o   bf16 [128][1024] = proj_o.weight         bias_o      fp32 [128]
 *
 * m: [B][S][N][64] of m_dtype; mask: uint8; out: [B][N][N][128] of out_dtype.
 * Workspace: b200_opm_workspace_bytes(S, N) bytes, 1024-byte aligned.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
  const void* w_ab;
  const void* w_o;
  const float* ln_w;
  const float* ln_b;
  const float* bias_o;
} b200_opm_weights;

size_t b200_opm_workspace_bytes(int S, int N);

int b200_opm_fwd(const void* m, const uint8_t* mask, int mask_ndim, void* out, const b200_opm_weights* w, int B,
                 int S, int N, int m_dtype, int out_dtype, void* workspace, size_t workspace_bytes,
                 b200_stream_t stream);

/* Partial form for callers that shard the MSA depth and the pair columns (DistributedOuterProductMean,
 * src/bioemu2/context_parallel/ops/outer_product_mean.py:116-262): m[S][N][64] holds only this caller's MSA rows,
 * the output is out[N][nj][128] for token columns j0 .. j0+nj-1, scaled by the device scalar *scale (1 / global
 * number of valid MSA rows) and, with add_bias = 0, without proj_o's bias -- partial results of different MSA
 * slices are summed by the caller and exactly one of them should carry the bias.  mask: uint8 [S][N].
 * Workspace: b200_opm_workspace_bytes(S, N). */
int b200_opm_cols_fwd(const void* m, const uint8_t* mask, void* out, const b200_opm_weights* w, int S, int N, int j0,
                      int nj, const float* scale, int add_bias, int m_dtype, int out_dtype, void* workspace,
                      size_t workspace_bytes, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Attention core on already projected operands: the fp32 softmax(q.k + bias, key mask) v section of
 * AttentionPairBias.forward (src/bioemu2/biomoa/ops/attention_pair_bias.py:165-222) and the core of the
 * context-parallel flash kernel (src/bioemu2/context_parallel/ops/triton/flash_attn_impl.py:9-228).
 * b200_apb_fwd and b200_triatt_fwd call it internally; it is exported for hosts that do their own projections.
 *
 *   out[b, q, h*dh_out + d] = sigmoid(gate[...]) * sum_k softmax_k(Q[b,q,h,:].K[b,k,h,:] + bias[b/bias_div, h, q, k]) V[b,k,h,d]
 *
 * All operands bf16.  Q and K live in one row-major buffer qk[batch][N][qk_width]: head h of Q at columns
 * q_col0 + h*DH, of K at k_col0 + h*DH (DH = head_dim_padded, 32 or 64; pad columns zero).  Q and bias must be
 * pre-multiplied by log2(e) (Q also by 1/sqrt(head dim)).  vT[batch][H*DH][v_pitch] is V transposed (keys
 * contiguous).  bias[bias_groups*H][N][bias_pitch].  mask: one byte per key at
 * mask[(b / mask_div) * mask_row_stride + k * mask_key_stride]; masked keys get the finite logit -1e6.
 * gate (raw logits, may be NULL) and out are addressed as base + b*batch_stride + q*pitch + col0 + h*dh_out + d.
 * N <= 8192.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
  const void* qk;
  int64_t qk_width, qk_batch_stride;
  int q_col0, k_col0;
  const void* vT;
  int64_t v_pitch;
  const void* bias;
  int64_t bias_pitch;
  int bias_groups, bias_div;
  const uint8_t* mask;
  int mask_div;
  int64_t mask_row_stride, mask_key_stride;
  const void* gate;
  int64_t gate_batch_stride;
  int gate_pitch, gate_col0;
  void* out;
  int64_t out_batch_stride;
  int out_pitch, out_col0;
  int head_dim_padded, head_dim_out;
  int N, H, batch;
} b200_attention_core_args;

int b200_attention_core_fwd(const b200_attention_core_args* args, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Single-track attention with pair bias, AttentionPairBias.forward
 * (src/bioemu2/biomoa/ops/attention_pair_bias.py:128-225):
 *   s' = LN(s) (if initial_norm);  q = Wq s' + b_q, k, v;  g = sigmoid(Wg s');  bias = proj_z(LN_z(z));
 *   o = softmax(q.k / sqrt(dh) + bias, masked keys replaced by -1e6) v;  out = Wo (g * o)
 * with the pair bias and key mask shared by the M ("multiplicity") copies of each batch element.
 * H <= 16 heads, head dim dh = c_s / H a multiple of 8 and <= 64; c_z = 128.  Heads are padded to
 * DH = 32 (dh <= 32) or 64 columns inside the packed weights:
 *
 *   w_qkg  bf16 [2*H*DH + c_s][c_s]  rows h*DH + d (d < dh) = Wq[h*dh + d] * log2(e)/sqrt(dh), zero rows for
 *                                    d >= dh; then the same for Wk (unscaled); then Wg
 *   b_qkg  fp32 [2*H*DH + c_s]       proj_q_bias in the q rows with the same scaling, zero elsewhere
 *   w_v    bf16 [H*DH][c_s]          Wv, head-padded
 *   w_z    bf16 [16][128]            proj_z.weight, zero rows for h >= H
 *   ln_z_w fp32 [128]; ln_z_b fp32 [128] or NULL (norm_z has no bias by default)
 *   ln_s_w, ln_s_b fp32 [c_s], both NULL when initial_norm is False
 *   w_o    bf16 [c_s][c_s]
 *
 * s, out: [B*M][N][c_s] of s_dtype; z: [B][N][N][128] of z_dtype; mask: uint8 [B][N].
 * Workspace: b200_apb_workspace_bytes(B, M, N, c_s, H) bytes, 1024-byte aligned.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
  const void* w_qkg;
  const float* b_qkg;
  const void* w_v;
  const void* w_z;
  const float* ln_z_w;
  const float* ln_z_b;
  const float* ln_s_w;
  const float* ln_s_b;
  const void* w_o;
} b200_apb_weights;

size_t b200_apb_workspace_bytes(int B, int M, int N, int c_s, int H);

int b200_apb_fwd(const void* s, const void* z, const uint8_t* mask, void* out, const b200_apb_weights* w, int B,
                 int M, int N, int c_s, int H, int s_dtype, int z_dtype, void* workspace, size_t workspace_bytes,
                 b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Triangle attention around the starting (ending = 0) or ending (ending = 1) node, 4 heads x 32, c_z = 128.
 * This op has NO counterpart in the reference (its trunk removed triangle attention,
 * src/bioemu2/biomoa/modules/pairmixer.py:459-462); it is the AlphaFold-2 algorithm with the reference's
 * pair-bias-attention conventions (bias-free projections except the gate, masked logits replaced by -1e6):
 *   h = LN(x);  q, k, v = W h;  bias[j,k] = W_b h[j,k];  g = sigmoid(W_g h + b_g)
 *   o[i,j] = softmax_k(q[i,j].k[i,k]/sqrt(32) + bias[j,k], keys masked by mask[i,k]) v[i,k];  out = W_o (g * o)
 * with x = z (starting node) or x = z transposed in its two token axes (ending node, result transposed back).
 *
 *   w_qkgv bf16 [512][128]: rows 0..127 W_q * log2(e)/sqrt(32), 128..255 W_k, 256..383 W_g, 384..511 W_v
 *   g_bias fp32 [128];  w_b bf16 [16][128] (rows 0..3 = W_b, rest zero);  w_o bf16 [128][128];  ln_w, ln_b fp32 [128]
 *
 * z, out: [B][N][N][128] of z_dtype; mask: uint8 [B][N][N].  With add_residual the result is z + update.
 * `out` may alias `z`: z is fully consumed by the projection stage before the output stage writes.
 * Workspace: b200_triatt_workspace_bytes(N) bytes, 1024-byte aligned.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
  const void* w_qkgv;
  const float* g_bias;
  const void* w_b;
  const void* w_o;
  const float* ln_w;
  const float* ln_b;
} b200_triatt_weights;

size_t b200_triatt_workspace_bytes(int N);

int b200_triatt_fwd(const void* z, const uint8_t* mask, void* out, const b200_triatt_weights* w, int B, int N,
                    int ending, int add_residual, int z_dtype, void* workspace, size_t workspace_bytes,
                    b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Pieces for sharded callers of the two attention ops (context-parallel wrappers,
 * src/bioemu2/context_parallel/ops/attention.py:45-105 and ops/attention_impl.py:558-706,984-1183).
 *
 * b200_pair_bias_fwd   out[h][line][pos] = log2(e) * proj(LN(z[line,pos]))[h] on a rectangular slab
 *                      z[n_rows][n_cols][128] (row pitch z_row_stride elements): the bias projection of
 *                      AttentionPairBias (w_z = proj_z, 16 x 128 zero padded) or of triangle attention (w_z = W_b).
 *                      (line, pos) = (row, column), or (column, row) with transposed = 1.  out is bf16 with element
 *                      strides out_plane (between heads) and out_pitch (between lines).
 * b200_apb_fwd_bias    b200_apb_fwd with the pair bias supplied by the caller: bias bf16 [B][H][N][bias_pitch] as
 *                      produced by b200_pair_bias_fwd (it may have been assembled from several GPUs' slabs).
 *                      Workspace as for b200_apb_fwd.
 * b200_triatt_slab_fwd triangle attention for `lines` complete attention rows: the slab z[n_rows][n_cols][128]
 *                      (contiguous) must span all columns for the starting node (lines = rows) or all rows for the
 *                      ending node (lines = columns); bias bf16 [4][tokens][bias_pitch] is the triangle bias of the
 *                      WHOLE pair tensor (transposed for the ending node), mask uint8 [n_rows][n_cols].
 *                      Workspace: b200_triatt_slab_workspace_bytes(n_rows, n_cols, ending).
 * ------------------------------------------------------------------------------------------------- */
int b200_pair_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w_z, void* out, int n_rows,
                       int n_cols, int64_t z_row_stride, int64_t out_plane, int64_t out_pitch, int H, int transposed,
                       int z_dtype, b200_stream_t stream);
int b200_apb_fwd_bias(const void* s, const void* bias, int64_t bias_pitch, const uint8_t* mask, void* out,
                      const b200_apb_weights* w, int B, int M, int N, int c_s, int H, int s_dtype, void* workspace,
                      size_t workspace_bytes, b200_stream_t stream);
size_t b200_triatt_slab_workspace_bytes(int n_rows, int n_cols, int ending);
int b200_triatt_slab_fwd(const void* z, const uint8_t* mask, const void* bias, int64_t bias_pitch, void* out,
                         const b200_triatt_weights* w, int n_rows, int n_cols, int ending, int add_residual, int z_dtype,
                         void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Single-track building blocks (token stream [rows][cols], rows = B*M*N): the pieces of
 * Transition.forward for widths other than 128/512 (src/bioemu2/biomoa/ops/transition.py:52-76) and of
 * ConditionedTransformerLayer.forward (src/bioemu2/biomoa/modules/transformer.py:26-53,317-353).
 *
 * b200_rows_to_bf16      y = [silu]([LN](x) * w + b) as bf16; normalize = 0 only converts.  w/b may be NULL.
 * b200_linear_bf16       out = x w^T [+ bias] [+ residual]; x bf16 [rows][in], w bf16 [out][in] (nn.Linear
 *                        layout), out/residual [rows][out] of out_dtype (residual may alias out).
 * b200_swiglu_fwd        h = silu(h12[:, :hidden]) * h12[:, hidden:], bf16.
 * b200_adaln_fwd         y = lns * (LN(x) * (1 + alpha) + beta), no learned affine (ada_ln, transformer.py:26-41);
 *                        alpha/beta are column blocks of the fp32 conditioning tensor cond[rows][cond_width].
 * b200_gated_residual_fwd  x += gamma * h in place (ada_scale + residual, transformer.py:349,352).
 * ------------------------------------------------------------------------------------------------- */
int b200_rows_to_bf16(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, int x_dtype,
                      int normalize, int silu, b200_stream_t stream);
int b200_linear_bf16(const void* x, const void* w, const float* bias, const void* residual, void* out, int64_t rows,
                     int in_features, int out_features, int out_dtype, b200_stream_t stream);
int b200_swiglu_fwd(const void* h12, void* h, int64_t rows, int hidden, b200_stream_t stream);
int b200_adaln_fwd(const void* x, const float* cond, int cond_width, int alpha_col, int beta_col, float lns, void* y,
                   int64_t rows, int cols, int x_dtype, b200_stream_t stream);
int b200_gated_residual_fwd(void* x, const void* h, const float* cond, int cond_width, int gamma_col, int64_t rows,
                            int cols, int x_dtype, int h_dtype, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Sequence-trunk prologue, recycling and pairwise conditioning: the HBM-bound glue around the pair blocks.
 *
 * b200_pair_outer_sum   z[i][j][:] = a[i][:] + c[j][:] (+ extra[i][j][:]), fp32: the pair initialisation
 *                       z_init_1(s_inputs)[:, :, None] + z_init_2(s_inputs)[:, None, :] plus the pair terms of the
 *                       feature encoders (src/bioemu2/biomoa/modules/pairmixer.py:231-250).  One batch item per call.
 * b200_add_rows         out[r][:] = x[r][:] + y[r % period][:], x/out fp32 (out may be x), y fp32 or bf16: the residual
 *                       of the unconditional branch (pairmixer.py:268) with period = rows, and the broadcast of
 *                       s_proj(emb) over the MSA rows (pairmixer.py:598) with period = tokens.
 * b200_rows2_to_bf16    y = LN(x1[r] | x2[r]) * w + b as bf16 [rows][cols1 + cols2]: LayerNorm over the concatenation
 *                       of two row sources that is never materialised - cat(z_trunk, token_rel_pos_feats) of
 *                       PairwiseConditioning.forward (src/bioemu2/biomoa/modules/diffusion.py:526-529).
 * The recycling update z_init + z_recycle(z_norm(z)) (pairmixer.py:282-283) is b200_rows_to_bf16 followed by
 * b200_linear_bf16 with z_init as the residual.
 * ------------------------------------------------------------------------------------------------- */
int b200_pair_outer_sum(const float* a, const float* c, const float* extra, float* z, int n_i, int n_j, int cols,
                        b200_stream_t stream);
int b200_add_rows(const float* x, const void* y, float* out, int64_t rows, int64_t period, int cols, int y_dtype,
                  b200_stream_t stream);
int b200_rows2_to_bf16(const void* x1, int cols1, const void* x2, int cols2, void* y, const float* w, const float* b,
                       int64_t rows, int x_dtype, int normalize, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Sliding-window attention with pair bias for the atom transformer, AttentionPairBiasSlidingWindow.forward
 * (src/bioemu2/biomoa/ops/attention_pair_bias.py:283-340): a query window of W atoms attends to the Hk keys centred
 * on it; keys beyond the ends of the sequence are zero rows and masked.  The projections around the core are
 * b200_rows_to_bf16 (norm_s) and b200_linear_bf16 (proj_qkv with proj_q_bias on the q columns, proj_g, proj_o).
 *
 * b200_window_bias_fwd       bias[win][h][i][j] = proj_z(norm_z(z[win][i][j][:]))[h] (:314), fp32; z fp32 or bf16
 *                            [windows][W][Hk][c_z], w_z fp32 [heads][c_z], ln_b may be NULL.
 * b200_window_attention_fwd  out = sigmoid(gate) * softmax_j(q.k_j / sqrt(d) + bias, masked keys REPLACED by -1e6) v
 *                            (:320-337) in fp32 arithmetic.  qkv bf16 [B*M][NW*W][3*heads*d] (q | k | v), gate / out
 *                            bf16 [B*M][NW*W][heads*d], bias fp32 [B][NW][heads][W][Hk] shared by the M samples of a
 *                            batch item, mask one byte per atom [B][NW*W].  d is 16, 32 or 64.
 * ------------------------------------------------------------------------------------------------- */
int b200_window_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const float* w_z, float* bias,
                         int64_t windows, int W, int Hk, int c_z, int heads, int z_dtype, b200_stream_t stream);
int b200_window_attention_fwd(const void* qkv, const void* gate, const float* bias, const uint8_t* mask, void* out, int B,
                              int M, int NW, int W, int Hk, int heads, int head_dim, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Pair-weighted averaging, PairWeightedAveraging.forward (src/bioemu2/biomoa/ops/pair_weighted_averaging.py:121-153),
 * is assembled from b200_rows_to_bf16 (norm_m), b200_linear_bf16 (proj_g, proj_o), b200_pair_bias_fwd (proj_z(norm_z(z))),
 * b200_bmm_nt (proj_m written transposed per head; the weighted average itself) and the two kernels below.
 *
 * b200_masked_softmax_rows  w[h][i][j] = softmax_j(mask[i][j] ? logits[h][i][j] : -1e6) (:141-142); logits bf16 in base-2
 *                           units [H][n_rows][pitch] as b200_pair_bias_fwd writes them, mask one byte per pair
 *                           [n_rows][n], w bf16 [H][n_rows][pitch] with zeros in columns n .. pitch-1.  n_rows == n
 *                           for the whole weight matrix; a rank of a context-parallel grid passes the rows it owns.
 * b200_pwa_gate             og[(s,i)][h*32+d] = sigmoid(g[(s,i)][h*32+d]) * o[h][i][s*32+d] (:145-151): gating and the
 *                           re-layout from per-head products to MSA rows; heads of 32 channels.
 * ------------------------------------------------------------------------------------------------- */
int b200_masked_softmax_rows(const void* logits, const uint8_t* mask, void* out, int H, int n_rows, int n, int pitch,
                             b200_stream_t stream);
int b200_pwa_gate(const void* o, const void* g, void* og, int S, int n, int H, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * fp32-accurate ("ieee") arithmetic.  The reference keeps some products in fp32 whatever the autocast state -- the
 * attention core (src/bioemu2/biomoa/ops/attention_pair_bias.py:165-167), the outer-product contraction
 * (outer_product_mean.py:66-74, matmul_precision "ieee"), the whole denoiser (biomoa/models/score_model.py:355) -- and
 * its fp32 tests hold the variants to 1e-6 .. 2e-6 (tests/biomoa/ops/test_triangle_multiplication.py:19-48).  On the
 * bf16 tensor cores an fp32 value travels as hi = bf16(x), lo = bf16(x - hi); with one operand laid out along K as
 * (hi | hi | lo) and the other as (hi | lo | hi), the ordinary K-major product of width 3K is hi.hi + hi.lo + lo.hi,
 * accumulated in fp32: b200_bmm_nt / b200_linear_bf16 serve unchanged (out_dtype fp32).
 *
 * b200_split_rows       y[r] = split([LayerNorm](x[r])): x fp32 [rows][cols] -> bf16 [rows][3*cols]; order 0 = hi|hi|lo
 *                       (the A side), 1 = hi|lo|hi (the B side, weights).  normalize != 0: LayerNorm with w, b (may be
 *                       NULL), eps, cols <= 1024.
 * b200_gate_rows_f32    out = a * sigmoid(b) (mode 0), silu(a) * b (mode 1) or a (mode 2), fp32, exact exponentials; a and b with
 *                       their own row pitches (elements); rowmask (one byte per row, may be NULL) zeroes masked rows.
 * b200_softmax_bias_f32 in place: s[g][q][:] = softmax_k(keymask[g / (H*bias_div)][k] ? s + bias[(g / (H*bias_div))*H + g % H][q][k] : -1e6)
 *                       for fp32 logits s[groups][n][n], g = (batch item * bias_div + copy) * H + head.
 * ------------------------------------------------------------------------------------------------- */
int b200_split_rows(const void* x, void* y, const float* w, const float* b, int64_t rows, int cols, float eps,
                    int normalize, int order, b200_stream_t stream);
int b200_gate_rows_f32(const float* a, int64_t a_pitch, const float* b, int64_t b_pitch, const uint8_t* rowmask,
                       float* out, int64_t rows, int cols, int mode, b200_stream_t stream);
int b200_softmax_bias_f32(float* s, const float* bias, const uint8_t* keymask, int64_t groups, int n, int H, int bias_div,
                          b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200PAIR_H_ */
