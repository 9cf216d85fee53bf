/* b200pf — C ABI of the B200 (sm_100a) Pairformer trunk kernels.
 *
 * The reference project (moritztng/tt-boltz, "TT-Bio") is pure Python and has no FFI; the
 * interface each entry point stands in for is therefore a Python call site of the reference's
 * device backend (tt_bio/tenstorrent.py) or of its CPU modules (tt_bio/reference.py,
 * tt_bio/boltz2.py).  Each declaration cites the call site it replaces.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device unless said otherwise;
 *   - no entry point allocates, frees or synchronises the device (unless stated); work is
 *     enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream);
 *   - return value: 0 on success, a negative B200PF_ERR_* code otherwise;
 *     b200pf_last_error() gives the message of the calling thread's last failure;
 *   - pair tensors use the reference layout: z[i][j][c], c contiguous, B = 1 folded away;
 *   - "planes" are channel-major bf16 matrices p[d][row][col] with a row pitch in elements
 *     (multiple of 8) and a plane stride in elements;
 *   - masks are uint8 (0 / 1), converted once by the host from the reference's float masks.
 */
#ifndef B200PF_H
#define B200PF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200PF_OK               0
#define B200PF_ERR_INVALID     -1   /* bad argument (null pointer, size, alignment)          */
#define B200PF_ERR_UNSUPPORTED -2   /* shape outside what the kernels are instantiated for   */
#define B200PF_ERR_CUDA        -3   /* a CUDA runtime / driver call failed                   */
#define B200PF_ERR_DEVICE      -4   /* a kernel reported a bounded wait that ran out         */

typedef uint16_t b200pf_bf16;       /* raw bfloat16 bits */

int         b200pf_version(void);
const char* b200pf_last_error(void);
/* Number of kernels this library has launched in the calling process (for benchmarks). */
long long   b200pf_launch_count(void);
/* Reads (and clears) the device status word kernels set when a bounded wait runs out.
 * Synchronises `stream`.  0 = clean; bit 1 = an mbarrier wait inside a kernel ran out, bit 2 = an index
 * check failed, bit 4 = a cross-rank barrier gave up waiting for a peer. */
int         b200pf_device_status(void* stream);

/* ------------------------------------------------------------------------------------------
 * fp32 validation tier: un-fused SIMT kernels, arithmetic in fp32 throughout.
 * Stand in for torch.nn.functional calls of the reference's CPU path.
 * ---------------------------------------------------------------------------------------- */

/* y[r][:] = LayerNorm(x[r][:]) * gamma + beta, eps 1e-5, biased variance.
 * Replaces nn.LayerNorm as used at tt_bio/reference.py:456, 467, 331 and tt_bio/boltz2.py:1241. */
int b200pf_f32_layernorm(const float* x, const float* gamma, const float* beta, float* y,
                         long long rows, int c, void* stream);

/* y[r][n] (+)= sum_k x[r][k] * w[n][k] (+ bias[n]); accumulate != 0 adds into y.
 * Replaces nn.Linear (tt_bio/boltz2.py:638-731) on the CPU path. */
int b200pf_f32_linear(const float* x, const float* w, const float* bias, float* y,
                      long long rows, int k, int n_out, int accumulate, void* stream);

/* Element-wise gates over [rows][c]; row_mask (may be NULL) has one byte per row.
 *   mode 0: y = a * sigmoid(b) * mask      (tt_bio/reference.py:458-461)
 *   mode 1: y = silu(a) * b                (tt_bio/boltz2.py:1244-1245)
 *   mode 2: y += a * sigmoid(b)            (tt_bio/reference.py:470 plus the residual :878) */
int b200pf_f32_gate(const float* a, const float* b, const uint8_t* row_mask, float* y,
                    long long rows, int c, int mode, void* stream);

/* t[i][j][c] = sum_k a[i][k][c] * b[j][k][c]   (incoming == 0, tt_bio/reference.py:467)
 * t[i][j][c] = sum_k a[k][i][c] * b[k][j][c]   (incoming != 0, tt_bio/reference.py:556)
 * a and b are [n][n][*] views with `in_pitch` floats between (row, col) positions; t is dense. */
int b200pf_f32_trimul_contract(const float* a, const float* b, float* t, int n, int d,
                               int in_pitch, int incoming, void* stream);

/* Softmax attention with additive mask and bias, fp32 (tt_bio/boltz2.py:790-810 and :357-364).
 *   logit[r][h][q][k] = scale * <Q[r][q][h], K[r][k][h]> (+) mask term (+) bias[h][q][k]
 *   mask term = -inf_value * (1 - mask[r*mask_rs + k*mask_ks]);
 *   order 0 adds the mask term first, then the bias (triangle attention);
 *   order 1 adds the bias first, then the mask term (single-track attention).
 * Q/K/V/O element (r, pos, h, e) lives at ptr[r*rs + pos*ps + h*hd + e]. */
int b200pf_f32_attention(const float* q, const float* k, const float* v, float* o,
                         const float* bias, long long bias_hs, long long bias_qs, long long bias_ks,
                         const uint8_t* mask, long long mask_rs, long long mask_ks,
                         int batch, int n_q, int n_k, int heads, int hd,
                         long long rs, long long ps, float scale, float inf_value, int order,
                         void* stream);

/* Linear with the result written transposed: yt[n][r] = sum_k x[r][k] w[n][k] (+ bias[n]), rows of yt are
 * yt_pitch floats apart.  Used to lay K and V out key-contiguous for the single-track attention. */
int b200pf_f32_linear_t(const float* x, const float* w, const float* bias, float* yt, long long yt_pitch,
                        long long rows, int k, int n_out, void* stream);

/* b200pf_f32_gate (modes 0-2, no row mask) on operands with separate row pitches (in floats). */
int b200pf_f32_gate_strided(const float* a, long long a_pitch, const float* b, long long b_pitch, float* y, long long y_pitch,
                            long long rows, int c, int mode, void* stream);

/* Single-track attention of AttentionPairBias (tt_bio/boltz2.py:357-366) in fp32, head dim 24:
 *   o[q][h] = sigmoid(g[q][h]) * softmax_k( scale * <q[q][h], k[k][h]> + bias[h][q][k] - inf * (1 - mask[k]) ) v[k][h]
 * q, g, o are row-major with their own pitches (head h at columns h*24 ..); k and v come transposed,
 * kt[(h*24 + e)][key] with kt_pitch floats per row (as b200pf_f32_linear_t writes them); g may be NULL.
 * With kt, vt and bias 16-byte aligned and kt_pitch, bias_hs, bias_qs multiples of 4 the tensor-core kernel runs
 * (3xTF32 products, key tiles of 64 staged through shared memory, one-pass softmax); otherwise a SIMT kernel that
 * loads its operands directly (slower; the two agree to fp32 rounding). */
int b200pf_f32_sattention(const float* q, long long q_pitch, const float* g, long long g_pitch,
                          const float* kt, const float* vt, long long kt_pitch, float* o, long long o_pitch,
                          const float* bias, long long bias_hs, long long bias_qs, const uint8_t* mask,
                          int n_q, int n_k, int heads, int hd, float scale, float inf_value, void* stream);

/* dst[j][i][:] (+)= src[i][j][:] for an [n][n][c] tensor (tt_bio/reference.py:326-328, 362-363). */
int b200pf_f32_transpose01(const float* src, float* dst, int n, int c, int accumulate, void* stream);

/* out[h][r] = sum_c LayerNorm(z[r][:])[c] * w[h][c]  (heads <= 16), fp32, one pass over z.
 * Replaces proj_z = LayerNorm -> Linear(c_z -> heads) -> 'b i j h -> b h i j'
 * (tt_bio/boltz2.py:331-337; device form tt_bio/tenstorrent.py:755-769) and the triangle bias
 * projection (tt_bio/reference.py:338-341).  `out_hs` = elements between heads. */
int b200pf_ln_proj_heads(const float* z, const float* gamma, const float* beta, const float* w,
                         float* out, long long out_hs, long long rows, int c, int heads, void* stream);

/* ------------------------------------------------------------------------------------------
 * bf16 tier: fused kernels.  z stays fp32 in HBM (the residual stream); operands are bf16,
 * accumulation fp32.  c_z = hidden = 128, 4 heads x 32 for triangle attention.
 * `rows` is the number of z rows [i] held locally (== n on one GPU); `n` is the full token count.
 * ---------------------------------------------------------------------------------------- */

/* Weight packing for the fused kernels is done once by the host (tt_boltz_b200/weights.py):
 * LayerNorm gains are folded into the bf16 weight rows, LayerNorm offsets become fp32 bias
 * vectors (W beta), and rows are re-ordered so that values a thread combines (p with g, fc1 with
 * fc2) land in the same thread.  The layouts are stated at each entry point. */

/* Triangle-multiplication producer: LN_in -> [p_in | g_in] projection -> p*sigmoid(g) -> mask
 * -> a/b written channel-major.  Replaces tt_bio/tenstorrent.py:410-452 (reference.py:456-464).
 *   z: fp32 [rows][n][128];  mask: [rows][n];
 *   the LayerNorm affine (ln_gamma, ln_beta: fp32 [128]) is applied in the kernel;
 *   w_pg bf16 [512][128] = 0.5 * (p_in rows of a, g_in rows of a, p_in rows of b, g_in rows of b),
 *   128 each (the halves turn p*sigmoid(g) into p' + p'*tanh(g'));
 *   incoming == 0: a[d][r][k] = u_a[r][k][d]  (plane rows = local z rows, cols = k)
 *   incoming != 0: a[d][c][r] = u_a[r][c][d]  (plane rows = z columns, cols = local z rows) */
typedef struct b200pf_plane_out {
    void*     ptr;            /* bf16 planes to write                                              */
    long long plane_stride;   /* elements between channels                                         */
    long long group_stride;   /* elements between groups of plane rows (unused when row_group <= 0) */
    int       row_group;      /* plane rows per group; <= 0: one group (plain [d][row][col] planes) */
} b200pf_plane_out;
/* element (d, row, col) of an output operand is written to
 *   ptr[(row / row_group) * group_stride + d * plane_stride + (row % row_group) * pitch + col];
 * row groups let a rank lay its planes out as one contiguous block per destination rank. */
int b200pf_trimul_producer(const float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                           const b200pf_bf16* w_pg, const b200pf_plane_out* a_out, const b200pf_plane_out* b_out,
                           int pitch, int rows, int n, int incoming, void* stream);

/* Operand description for the contraction: element (seg, d, row, col) of an operand lives at
 * ptr[seg*seg_stride + d*plane_stride + row*pitch + col]. */
typedef struct b200pf_planes {
    const void* ptr;
    long long   plane_stride;   /* elements between channels d                              */
    long long   seg_stride;     /* elements between segments (ignored when nseg == 1)       */
    int         pitch;          /* elements between rows; multiple of 8                     */
    int         rows;           /* rows per segment                                         */
    int         cols;           /* valid columns (contraction index) per segment            */
    int         nseg;           /* number of segments                                       */
    int         seg_is_k;       /* 1: segments split the contraction index; 0: split rows   */
} b200pf_planes;

/* x[d][i][j] = sum_k A[d][i][k] * B[d][j][k] for d < channels: the N x N x N contraction of
 * the triangle multiplication as a batched K-major GEMM (tcgen05 + TMEM, TMA-fed).
 * Replaces the per-chunk ttnn.matmul at tt_bio/tenstorrent.py:453-460 (reference.py:467, 556).
 * x is bf16 planes x[d][i][j] with pitch x_pitch; with x_row_group > 0 the output rows are written
 * in groups, element (d, i, j) at (i / x_row_group) * x_group_stride + d * x_plane_stride +
 * (i % x_row_group) * x_pitch + j, so that a rank that contracts a slice of the channels for every
 * row can send each owner of output rows one contiguous block.  Both operands may be segmented
 * along rows or along the contraction index (segments of 128-row multiples / 64-column multiples).
 * variant 0 = tcgen05 bf16, 2 = tcgen05 block-scaled MXFP8: a / b are byte planes of e4m3
 * values (pitch, plane_stride, seg_stride in bytes, multiples of 16; k segments multiples of 128 columns)
 * and a_scales / b_scales their e8m0 scale blocks as written by b200pf_trimul_producer_mx; for a segmented
 * operand the scale buffers of the segments, each b200pf_mx_scale_bytes(rows, cols, channels) long for the
 * rows / cols of ONE segment, lie one behind the other in segment order (which is what an all-to-all of the
 * producer's channel-major scale blocks delivers).  The scales are ignored by variant 0. */
int b200pf_trimul_contract(const b200pf_planes* a, const b200pf_planes* b,
                           const void* a_scales, const void* b_scales,
                           b200pf_bf16* x, long long x_plane_stride, int x_pitch,
                           int x_row_group, long long x_group_stride,
                           int channels, int variant, void* stream);

/* The bf16 contraction with both output indices regrouped: element (d, row, col) is written to
 *   (row / x_row_group) * x_group_stride + d * x_plane_stride + (row % x_row_group) * x_pitch
 *   + (col / x_col_group) * x_colgroup_stride + col % x_col_group
 * (x_row_group <= 0: rows not grouped; x_col_group a multiple of 32; unsegmented operands).  Used where the consumer
 * of a GEMM wants its output in another index order than [row][col] (MSA stack). */
int b200pf_gemm_grouped(const b200pf_planes* a, const b200pf_planes* b, b200pf_bf16* x, long long x_plane_stride,
                        int x_pitch, int x_row_group, long long x_group_stride, int x_col_group,
                        long long x_colgroup_stride, int channels, void* stream);

/* MXFP8 form of the producer (the counterpart of the reference's block-fp8 "fast" mode,
 * tt_bio/tenstorrent.py:178-181, 432-452): same computation as b200pf_trimul_producer, but
 * a / b are quantised straight from fp32 to e4m3 with one e8m0 scale per 32 elements along the
 * contraction index (scale = smallest power of two with amax / scale <= 448).
 *   a_out / b_out: byte planes [128][plane rows][pitch] (pitch, plane_stride in bytes, multiples of 16);
 *   a_scales / b_scales: b200pf_mx_scale_bytes(plane rows, plane cols, 128) bytes each, zeroed once by
 *   the caller; 512-byte blocks, block = (d * ceil(cols/128) + k/128) * row_blocks + row/128 with
 *   row_blocks = 2*ceil(rows/256), byte in block = (row%32)*16 + ((row%128)/32)*4 + (k/32)%4. */
long long b200pf_mx_scale_bytes(int rows, int cols, int channels);
int b200pf_trimul_producer_mx(const float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                              const b200pf_bf16* w_pg, uint8_t* a_out, uint8_t* b_out, uint8_t* a_scales,
                              uint8_t* b_scales, long long plane_stride, int pitch, int rows, int n, int incoming,
                              void* stream);
/* Expand MXFP8 planes to bf16 planes (exact).  Cross-check of the block-scaled contraction and a way to feed MXFP8
 * operands to consumers that want bf16. */
int b200pf_mx_dequant(const uint8_t* planes, const uint8_t* scales, b200pf_bf16* out, long long plane_stride,
                      int pitch, long long out_plane_stride, int out_pitch, int rows, int cols, int channels,
                      void* stream);

/* Triangle-multiplication epilogue: z += (LN_out(x) W_pout^T) * sigmoid(LN_in(z) W_gout^T), on tcgen05.
 * Replaces tt_bio/tenstorrent.py:463-502 plus the residual add :1007-1011.
 * x planes as written by the contraction; x is multiplied RAW as an MN-major operand
 * straight from its planes; the LayerNorm over the channels of x is applied after the GEMM per
 * position (mean / rstd from the tile), the update leaves through TMA reduce-add into z.
 *   w_pout: bf16 [128][128] = 0.5 * W_pout * gamma_out;  wsum: fp32 [128] row sums of that bf16 matrix;
 *   wb: fp32 [128] = 0.5 * W_pout beta_out;  w_gout: bf16 [128][128] = 0.5 * W_gout;
 *   ln_in_gamma / ln_in_beta: fp32 [128] LayerNorm of z for the gate, applied in the kernel. */
int b200pf_trimul_epilogue_tc(float* z, const b200pf_bf16* x, long long x_plane_stride, int x_pitch,
                              const float* ln_in_gamma, const float* ln_in_beta,
                              const b200pf_bf16* w_pout, const b200pf_bf16* w_gout,
                              const float* wsum, const float* wb, int rows, int n, void* stream);

/* Triangle-attention producer: LN -> [q|k|v|g] projection and the 4-head triangle bias.
 * Replaces tt_bio/tenstorrent.py:545-567, 603-614 (reference.py:331-341, 99-120).
 *   z is viewed as [rows][n][128] (a row shard, or a column shard stored [i][j_local][128]);
 *   LN affine from ln_gamma / ln_beta (fp32 [128]); w_qkgv bf16 [512][128] = q rows (scaled by
 *   log2(e)/sqrt(32)), k, 0.5 * g, v rows; w_bias_f32: fp32 [4][128] bias rows times log2(e);
 * A "line" is a row of the view (ending == 0, positions = its n columns) or a column of the view
 * (ending != 0, positions = its `rows` rows).  Outputs (bf16):
 *   q,k: [line][pos][head][32];  v: transposed, [line][head][32][vt_pitch] (positions contiguous), as the
 *          attention core reads it;
 *   g:     sigmoid(gate) in the layout of the view, [rows][n][128];
 *   tri_bias: element (head, line, pos) at tri_bias[head*bias_hs + line*bias_qs + pos]: the bias
 *          of query `line` and key `pos` (for the ending node that is beta[row pos][col line]). */
int b200pf_triatt_producer(const float* z, const float* ln_gamma, const float* ln_beta, const float* w_bias_f32,
                           const b200pf_bf16* w_qkgv,
                           b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                           b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                           int vt_pitch, int rows, int n, int ending, void* stream);
/* The same producer reading the pair tensor in bf16 (same view), as it arrives from the sharded exchange. */
int b200pf_triatt_producer_bf16z(const b200pf_bf16* z, const float* ln_gamma, const float* ln_beta, const float* w_bias_f32,
                           const b200pf_bf16* w_qkgv,
                           b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                           b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                           int vt_pitch, int rows, int n, int ending, void* stream);

/* Fused flash-style triangle attention on tcgen05 / TMEM: for each line and head, softmax(q k^T + mask + bias) v
 * with online softmax in the log2 domain; logits never leave the SM.  Replaces the SDPA call at
 * tt_bio/tenstorrent.py:569-572 (reference.py:343-360, boltz2.py:790-810).
 * S = Q K^T and O = P V run as tcgen05.mma with accumulators in TMEM, operands come in by TMA; four lines per
 * CTA (four softmax groups in flight, one thread per query row), the bias tile fetched once for the four and
 * multiplied in once per pair of lines; masked keys get -1e9 (times log2 e); the running output stays in TMEM and
 * is rescaled only when a row maximum has grown by more than 2^8.
 *   n = queries = keys per line;  q, k: [line][pos][head][32] (as written by the producer); vt: v transposed
 *   [line][head][32][vt_pitch];  bias element (head, query, key) at bias[head*bias_hs + query*bias_qs + key];
 *   mask_lines: uint8 [lines][mask_pitch] (1 = attend), one contiguous row per line, mask_pitch a
 *   multiple of 16 covering n rounded up to 64 (the host transposes the mask for the ending node);
 *   o element (line, pos, c) at o[line*o_line_stride + pos*o_pos_stride + c]. */
int b200pf_triatt_core_tc4(const b200pf_bf16* q, const b200pf_bf16* k, const b200pf_bf16* vt, int vt_pitch,
                           const b200pf_bf16* bias, long long bias_hs, long long bias_qs,
                           const uint8_t* mask_lines, int mask_pitch,
                           b200pf_bf16* o, long long o_line_stride, long long o_pos_stride,
                           int lines, int n, void* stream);

/* Triangle-attention epilogue: z += (o * g) W_o^T  (g already passed through the sigmoid).
 * Replaces tt_bio/tenstorrent.py:580-591 and the residual :1013-1021 (reference.py:122-136). */
int b200pf_triatt_epilogue(float* z, const b200pf_bf16* o, const b200pf_bf16* g,
                           const b200pf_bf16* w_o, long long n_rows_flat, void* stream);
/* The same product stored instead of added: upd = (o * g) W_o^T in bf16, [n_rows_flat][128].  The sharded ending node
 * uses it to send the update, not the whole fp32 tensor, back to the row owners. */
int b200pf_triatt_epilogue_update(b200pf_bf16* upd, const b200pf_bf16* o, const b200pf_bf16* g,
                                  const b200pf_bf16* w_o, long long n_rows_flat, void* stream);

/* Pair transition: z += W3( silu(W1 LN(z)) * (W2 LN(z)) ), hidden 512 kept on chip, on tcgen05.
 * Replaces tt_bio/tenstorrent.py:869-946 and the residual :1023-1025 (boltz2.py:1241-1246).
 * GEMM1 per 64-channel chunk of the hidden layer into
 * TMEM, SwiGLU in registers, hidden activations written back to TMEM as the A operand of GEMM2,
 * update through TMA reduce-add into z; weights streamed from L2 by TMA.
 *   ln_gamma / ln_beta: fp32 [128], applied in the kernel;
 *   w12: bf16 [8][128][128]: per chunk c the rows 0.5 * fc1[64c .. 64c+63] then fc2[64c .. 64c+63];
 *   w3:  bf16 [8][128][64]: per chunk the matching 64 columns of fc3. */
int b200pf_transition_z_tc(float* z, const float* ln_gamma, const float* ln_beta,
                           const b200pf_bf16* w12, const b200pf_bf16* w3, long long n_rows_flat, void* stream);

/* Triangle multiplication (producer -> contraction -> epilogue, bf16 tier) for callers that cannot
 * allocate device memory.  No counterpart in the reference.
 * Why it exists: the three stages pass their a / b / x planes through global memory, which the
 * caller normally provides.  A host that runs inside a fixed memory budget, inside a callback
 * where the allocator may not be entered, or in a server that forbids allocation after start-up
 * has nowhere to get those planes from; here they live in a 12 MiB array that is part of the
 * library image on every GPU that loads it (held until the process exits).
 *   - limit: n <= 128 tokens; larger n is refused with B200PF_ERR_UNSUPPORTED and a message;
 *   - z (fp32 [n][n][128]) is updated in place; mask is [n][n]; weights as for the three stage
 *     tcgen05 stage entry points (ln_gamma / ln_beta [128], w_pg [512][128], and w_pout / w_gout / wsum / wb as
 *     for b200pf_trimul_epilogue_tc);
 *   - the call itself never calls cudaMalloc / cudaFree or any allocating routine;
 *   - the first call on a device looks up the device address of the array (cudaGetSymbolAddress), and
 *     the three stages it runs raise their kernels' shared-memory limit and resolve the tensor-map
 *     encoder on their first use per device; the driver may also load the kernels lazily at the first
 *     launch.  So make one complete warm-up call per device before starting any stream capture and
 *     before calling from a context that must not enter the driver's loader (cudaDeviceReset
 *     invalidates the cached addresses: do not call again in that process after one);
 *   - all calls share the one array and it keeps the previous call's contents.  Nothing in it
 *     has to start at zero (each stage overwrites everything the next one reads), but two calls
 *     whose kernels overlap on the GPU (different streams) race on it: serialise them. */
int b200pf_tri_mul_noalloc(float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                           const b200pf_bf16* w_pg,
                           const b200pf_bf16* w_pout, const b200pf_bf16* w_gout,
                           const float* wsum, const float* wb,
                           int n, int incoming, void* stream);

/* ----------------------------------------------------------------------------------------
 * Outer-product mean: the MSA stack's write into the pair tensor, the step before the Pairformer
 * in every recycle.  Replaces OuterProductMean at tt_bio/tenstorrent.py:1632-1718 (reference.py:571-669):
 *   z[i][j][:] (+)= W_o vec(sum_s a[s][i][:] (x) b[s][j][:]) / max(1, sum_s mask[s][i] mask[s][j]) + bias,
 *   a = mask * LN(m) W_a^T, b = mask * LN(m) W_b^T;   m fp32 [S][N][64], mask uint8 [S][N], 32 channels per side.
 * Four stages: producer -> b200pf_opm_outer -> b200pf_trimul_contract (one channel, A = the outer products
 * [pairs][1024], B = W_o bf16 [128][1024]) -> finalize.  A caller bounds the memory of the outer products by
 * walking blocks of tokens i (n_i of them per call).
 * ---------------------------------------------------------------------------------------- */

/* LN + both projections + mask, written transposed as K-major GEMM operands:
 * a_t[(tok*32 + c)][s], b_t[(tok*32 + d)][s], bf16, `pitch` elements per row (>= s_len, multiple of 8; elements at
 * s >= s_len are not written and not read).  w_ab fp32 [64][64]: rows 0-31 proj_a.weight, rows 32-63 proj_b.weight. */
int b200pf_opm_producer(const float* m, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                        const float* w_ab, b200pf_bf16* a_t, b200pf_bf16* b_t, int s_len, int n, int pitch, void* stream);

/* x2[i][j][c][d] = sum_s a_t[(i, c)][s] * b_t[(j, d)][s] for n_i tokens i (a_t points at the first one's rows) and
 * all n_j tokens j: bf16 [n_i][n_j][32][32], fp32 accumulation (the contraction kernel of the triangle
 * multiplication with its output regrouped per token pair). */
int b200pf_opm_outer(const b200pf_bf16* a_t, const b200pf_bf16* b_t, b200pf_bf16* x2, int s_len, int n_i, int n_j,
                     int pitch, void* stream);

/* bits[tok][w]: bit b of word w = mask[w*32 + b][tok] != 0; (s_len + 31) / 32 words per token. */
int b200pf_opm_mask_bits(const uint8_t* mask, uint32_t* bits, int s_len, int n, void* stream);

/* z[il][j][:] = (accumulate ? z[il][j][:] : 0) + y[il*n + j][:] / count(i0 + il, j) + bias for il < n_i, j < n;
 * y bf16 [n_i*n][128] (the projected outer products), z fp32 rows of token i0 onwards, count from the mask bits
 * (at least 1).  At most 16384 sequences. */
int b200pf_opm_finalize(const b200pf_bf16* y, const uint32_t* bits, const float* bias, float* z, int s_len,
                        int i0, int n_i, int n, int accumulate, void* stream);

/* ----------------------------------------------------------------------------------------
 * Row kernels of the MSA stack (m fp32 [S][N][64]) around GEMMs run by b200pf_trimul_contract.  The token axis
 * of every bf16 operand is padded to np (a multiple of 8, >= n); padding rows are zero.
 *   pair-weighted averaging (tt_bio/tenstorrent.py:1542-1629, reference.py:672-800):
 *     ln = b200pf_msa_ln_bf16(m)                         [S*np][64]
 *     vg = b200pf_gemm_grouped(A = [proj_m ; proj_g] bf16 [512][64], B = ln) -> [16][S][32][np]: v groups 0-7 (heads),
 *          g groups 8-15; np a multiple of 32 here
 *     logits = b200pf_ln_proj_heads(z, norm_z, proj_z, 8 heads);  w = b200pf_pwa_softmax(logits, mask)
 *     o = contract over 8 heads (A = v as [8][S*32][np], B = w [8][n][pitch])   -> [8][S][32][np]
 *     val = b200pf_pwa_gate_transpose(o, g);  t = contract(A = val [S*np][256], B = proj_o bf16 [64][256]);
 *     b200pf_msa_add_rows(m, t)
 *   MSA transition (Transition(64, 256), tt_bio/boltz2.py:1188-1258):
 *     ln -> contract(A = ln, B = [fc1 ; fc2] bf16 [512][64]) -> b200pf_msa_swiglu -> contract(B = fc3 bf16 [64][256])
 *     -> b200pf_msa_add_rows
 * ---------------------------------------------------------------------------------------- */
int b200pf_msa_ln_bf16(const float* m, const float* gamma, const float* beta, b200pf_bf16* out, int s_len, int n, int np,
                       void* stream);
/* w[h][i][j] = softmax over j of logits[h][i][j] - inf_value * (mask[i][j] == 0); bf16 rows of `pitch`, zero beyond n. */
int b200pf_pwa_softmax(const float* logits, const uint8_t* mask, b200pf_bf16* w, int n, int pitch, int heads, float inf_value,
                       void* stream);
/* val[s*np + tok][head*32 + d] = o * sigmoid(g) at (head, s, d, tok): o, g bf16 [8][S][32][np] -> bf16 [S*np][256], the
 * K-major operand of the output projection. */
int b200pf_pwa_gate_transpose(const b200pf_bf16* o, const b200pf_bf16* g, b200pf_bf16* val, int s_len, int np, void* stream);
/* out[r][c] = silu(h[r][c]) * h[r][256 + c]: bf16 rows of 512 -> bf16 rows of 256. */
int b200pf_msa_swiglu(const b200pf_bf16* h, b200pf_bf16* out, long long rows, void* stream);
/* m[s][i][:] += t[s*np + i][:]  (t bf16 rows of 64). */
int b200pf_msa_add_rows(float* m, const b200pf_bf16* t, int s_len, int n, int np, void* stream);
/* m[s][i][:] += e[i][:] (fp32 rows of 64): the projected single representation added to every sequence's embedding
 * (MSAModule.forward, tt_bio/reference.py:1275-1276). */
int b200pf_msa_add_token_rows(float* m, const float* e, int s_len, int n, void* stream);

/* All-to-all of equal blocks over peer mappings (multi-GPU path, no counterpart in the reference, whose
 * cards do not exchange data: tt_bio/distributed.py fans whole jobs out).  Block t of `send` (world blocks
 * of block_bytes) is written to slot `rank` of rank t's receive buffer; recv_ptrs is a HOST array of the
 * world receive-buffer addresses as mapped in this process (symmetric memory, no multicast).  One launch per
 * rank; the caller puts a cross-rank barrier between this and the consumers of the receive buffer. */
int b200pf_peer_scatter(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                        int rank, int world, void* stream);
/* The same all-to-all for blocks that are strided on one or both sides (no counterpart in the reference either):
 * block t is `chunks` pieces of chunk_bytes; piece q is read at send + t * src_block_stride + q * src_chunk_stride
 * and written to rank t at recv_ptrs[t] + rank * dst_slot_stride + q * dst_chunk_stride (bytes, multiples of 16).
 * It is how the row-sharded pair tensor is turned into a column shard for the ending-node attention, and back,
 * without packing copies: rows -> columns reads nr pieces of nr * 128 elements out of every local row,
 * columns -> rows writes them straight into the receiver's row shard. */
int b200pf_peer_scatter_strided(const void* send, const unsigned long long* recv_ptrs, long long chunk_bytes, int chunks,
                                long long src_block_stride, long long src_chunk_stride,
                                long long dst_slot_stride, long long dst_chunk_stride, int rank, int world, void* stream);
/* All-gather form of the same: `send` is ONE block, written to slot `rank` of every rank's receive buffer. */
int b200pf_peer_broadcast(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                          int rank, int world, void* stream);
/* The exchanges with the barrier that normally follows them built in: the CTA that finishes last signals the
 * peers and waits for theirs, so one launch does what b200pf_peer_scatter + b200pf_peer_barrier do in two.
 * `channel` (0..7) picks the device-side CTA counter: exchanges that may run at the same time on one device
 * (different streams) must use different channels, and their signal pads and generations are per channel too. */
typedef struct b200pf_peer_sync {
    const unsigned long long* pad_ptrs;   /* HOST array: the world signal pads as mapped in this process */
    unsigned int generation;              /* grows by one per barrier of this channel, on every rank */
    long long    timeout_ns;              /* the wait gives up after this long: status bit 4, no trap */
    int          channel;
} b200pf_peer_sync;
int b200pf_peer_scatter_sync(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                             int rank, int world, const b200pf_peer_sync* sync, void* stream);
int b200pf_peer_broadcast_sync(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                               int rank, int world, const b200pf_peer_sync* sync, void* stream);
int b200pf_peer_scatter_strided_sync(const void* send, const unsigned long long* recv_ptrs, long long chunk_bytes, int chunks,
                                     long long src_block_stride, long long src_chunk_stride,
                                     long long dst_slot_stride, long long dst_chunk_stride, int rank, int world,
                                     const b200pf_peer_sync* sync, void* stream);
/* The strided exchange with fp32 -> bf16 narrowing on the way (the sharded ending-node attention sends z to the
 * column owners in bf16: the producer rounds its LayerNorm output to bf16 anyway).  Sizes and strides count ELEMENTS
 * (multiples of 8); `send` is fp32, the receive buffers hold bf16. */
int b200pf_peer_scatter_strided_f32_bf16_sync(const float* send, const unsigned long long* recv_ptrs, long long chunk_elems, int chunks,
                                              long long src_block_stride, long long src_chunk_stride,
                                              long long dst_slot_stride, long long dst_chunk_stride, int rank, int world,
                                              const b200pf_peer_sync* sync, void* stream);
/* z[i] += upd[i] for n_elems elements (bf16 update into the fp32 residual stream): the receiving end of an update
 * that crossed the wire in bf16. */
int b200pf_add_bf16(float* z, const b200pf_bf16* upd, long long n_elems, void* stream);
/* Cross-rank barrier of the peer-write exchanges (no counterpart in the reference: its cards never wait on
 * each other; the nearest thing is the job lease that expires when a worker stops reporting,
 * tt_bio/distributed.py:22, 214).  pad_ptrs is a HOST array of the world signal pads as mapped in this process
 * (each at least world 32-bit words, zero before the first barrier).  One tiny launch per rank: it stores
 * `generation` into slot `rank` of every rank's pad and waits until every slot of its own pad has reached
 * `generation`.  Generations must grow by one per barrier on every rank.  Enqueued after an exchange on the
 * same stream it means "my blocks have landed" to the peers and "all blocks for me have landed" to the kernels
 * behind it.  The wait gives up after timeout_ns: the kernel then sets bit 4 of the device status word
 * (b200pf_device_status) and returns; it never traps, and the context stays usable. */
int b200pf_peer_barrier(const unsigned long long* pad_ptrs, unsigned int generation, int rank, int world,
                        long long timeout_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200PF_H */
