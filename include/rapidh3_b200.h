/* librapidh3_b200 -- C ABI of the B200 (sm_100a) kernels behind the Rapid-H3 operator surface.
 *
 * Conventions
 *   - every entry point returns int: 0 = ok, < 0 = argument error, > 0 = a cudaError_t value;
 *     rh3_last_error_string() describes the last failure on the calling thread;
 *   - all pointers are DEVICE pointers unless stated otherwise; the caller owns every buffer,
 *     the library allocates nothing; work is enqueued on `stream` and never synchronised,
 *     except by rh3_check_status();
 *   - activations are bf16, codes are int8 or fp8-e4m3 bytes, scales fp32, row-major;
 *     strides are in elements of the tensor they describe;
 *   - "reference" citations are paths inside the jeet0733/Rapid-H3 repository.
 */
#ifndef RAPIDH3_B200_H_
#define RAPIDH3_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

#define RH3_KIND_I8 0 /* int8 x int8 -> int32 */
#define RH3_KIND_F8 1 /* e4m3 x e4m3 -> fp32 */

/* ---- library ------------------------------------------------------------------------------- */
const char* rh3_last_error_string(void);
int rh3_version(void);
int rh3_sm_count(void);
/* Synchronises `stream`, stores the device status word in *status_out (0 = every bounded device
 * wait completed; otherwise the code of the wait that gave up) and clears it. */
int rh3_check_status(cudaStream_t stream, int* status_out);
/* Self-test of the bounded device waits: launches one small CTA whose threads wait, for at most `max_polls`
 * polls (1 .. 2^20), on a barrier that nothing ever completes. The wait gives up, the kernel records status
 * 190 in the device status word (read it with rh3_check_status) and returns by itself; *left_normally (device
 * memory, one int) is set to 1 when every thread left through the give-up path. Nothing faults or hangs: this is
 * how the path "a wait ran out" of every kernel of the library is exercised. It has no counterpart in the
 * reference (whose kernels wait without a limit). */
int rh3_selftest_wait_expiry(int64_t max_polls, int* left_normally, cudaStream_t stream);
/* Issue-rate probe of the tensor pipe (no reference counterpart): every SM issues groups * 64 MMAs of 128 x 256 x 32
 * (kind 0 = int8, 1 = e4m3) or 128 x 256 x 16 (kind 2 = bf16) on shared-memory operands that are zero or, with
 * random_operands != 0, a fixed pseudo-random pattern (the switching activity of real data, which the power cap
 * responds to); the caller times the launch with CUDA events and divides *ops_out (operations of the launch) by it:
 * the retire rate of the MMAs under the clocks the GPU holds, the denominator of the 8-bit tensor rooflines.
 * pattern 0: 64 MMAs per commit; 1 and 2: the issue pattern of a pipelined GEMM main loop (four-stage ring: per four
 * MMAs a wait on the stage's barrier, the descriptors and a commit), descriptors rebuilt per stage (1) or kept in
 * registers (2), or with the whole warp in the loop and one elected lane issuing (3): what the issuing thread's own
 * instruction stream costs. pattern 4: pattern 0 with MMAs of 128 columns (half the work per instruction; *ops_out
 * counts accordingly): the rate of the narrow tiles of the 128-channel convolutions. */
int rh3_selftest_mma_rate(int kind, int64_t groups, int random_operands, int pattern, double* ops_out,
                          cudaStream_t stream);
/* The main loop of a 128 x 256 int8 GEMM tile without an epilogue, on every SM (no reference counterpart): a four-stage
 * ring; per stage a bulk copy of fill_bytes (0, 16384, 32768 or 49152) from src into shared memory, then four MMAs of
 * 128 x 256 x 32 on the stage. Timed by the caller; *ops_out = operations of the launch. It shows the MMA rate an SM
 * sustains while taking in fill_bytes per 512 tensor cycles: 49152 is what the GEMM's tile shape asks for. */
int rh3_selftest_mma_feed(const void* src, int64_t src_bytes, int64_t stages, int fill_bytes, double* ops_out,
                          cudaStream_t stream);

/* ---- per-token quantizers (HBM-bound) ------------------------------------------------------ */
/* q[M,K] int8, s[M] fp32: s = max(amax/127, 1e-12), q = clamp(rint(x/s), +-127).
 * Replaces kernels.quantize_rows(x, "int8_rowwise") (custom_nodes/rapid_h3/kernels.py:75-82) and
 * triton_fp8.quant_rows_i8 (custom_nodes/rapid_h3/triton_fp8.py:57-64). */
int rh3_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                      cudaStream_t stream);
/* q[M,K] fp8-e4m3, s = max(amax/448, 1e-12). Replaces kernels.quantize_rows(x, "fp8_rowwise")
 * (kernels.py:75-82) and triton_fp8.quant_rows (triton_fp8.py:449-455). */
int rh3_quant_rows_fp8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                       cudaStream_t stream);
/* One scale for the whole tensor: s = max(max|x| / 448, 1e-12), q = e4m3(x / s); the same s is written to every
 * entry of s[M], so the codes go through the row-scaled GEMM unchanged. `amax` is one fp32 word of device scratch
 * (written here: the tensor's max |x|). Two kernel launches. Replaces the "fp8_tensor" branches of
 * kernels.quantize_weight and kernels.linear (custom_nodes/rapid_h3/kernels.py:63-65,125-128). */
int rh3_quant_tensor_fp8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s, float* amax,
                         cudaStream_t stream);
/* x[M, 2F]: quantizes silu(x[:, :F]) * x[:, F:] to int8 [M, F].
 * Replaces triton_fp8.swiglu_rot_quant_rows_i8 without rotation (triton_fp8.py:437-439, prologue :137-139). */
int rh3_swiglu_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t F, void* q, int64_t ldq, float* s,
                             cudaStream_t stream);
/* o[H, M, 128] head-major (stride_h elements between heads) -> q[M, H*128] int8, no transpose copy.
 * Replaces triton_fp8.rot_quant_heads_i8 without rotation (triton_fp8.py:429-434, gather :134-135). */
int rh3_quant_heads_i8(const void* o, int64_t stride_h, int64_t H, int64_t M, void* q, int64_t ldq, float* s,
                       cudaStream_t stream);
/* Generalisation of rh3_quant_heads_i8 to groups of gw columns: o[G, M, gw] -> q[M, G*gw]. Used on the
 * output of the head-to-token exchange of sequence-parallel attention, which arrives grouped by source
 * rank. Same reference as rh3_quant_heads_i8. */
int rh3_quant_groups_i8(const void* o, int64_t stride_g, int64_t G, int64_t gw, int64_t M, void* q, int64_t ldq,
                        float* s, cudaStream_t stream);
/* y = rms_norm(x, eps) * w * (1 + scale[idx[m]]) + shift[idx[m]] -> int8 rows. w may be NULL.
 * shift/scale are fp32 tables with row stride ld_tab. Replaces triton_fp8.norm_mod_rot_quant_rows_i8
 * without rotation (triton_fp8.py:442-446, prologue :141-148, :165-172). */
int rh3_norm_mod_quant_rows_i8(const void* x, int64_t ldx, const void* w, float eps, const int32_t* idx,
                               const float* shift, const float* scale, int64_t ld_tab, int64_t M, int64_t K,
                               void* q, int64_t ldq, float* s, cudaStream_t stream);

/* The same four quantizers with the H256 ConvRot rotation (x . blockdiag(H256)^T over groups of 256 channels,
 * H256 = Kronecker powers of the regular 4x4 Hadamard matrix / 16) applied before the abs-max: the `int8_rot`
 * recipe, whose weights are stored as W . blockdiag(H256)^T. The rotated width must be a multiple of 256.
 * Replace triton_fp8.rot_quant_rows_i8 / swiglu_rot_quant_rows_i8 / rot_quant_heads_i8 /
 * norm_mod_rot_quant_rows_i8 (custom_nodes/rapid_h3/triton_fp8.py:424-446, rotation :70-112, :151-194). */
int rh3_rot_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                          cudaStream_t stream);
int rh3_swiglu_rot_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t F, void* q, int64_t ldq, float* s,
                                 cudaStream_t stream);
int rh3_rot_quant_groups_i8(const void* o, int64_t stride_g, int64_t G, int64_t gw, int64_t M, void* q, int64_t ldq,
                            float* s, cudaStream_t stream);
int rh3_norm_mod_rot_quant_rows_i8(const void* x, int64_t ldx, const void* w, float eps, const int32_t* idx,
                                   const float* shift, const float* scale, int64_t ld_tab, int64_t M, int64_t K,
                                   void* q, int64_t ldq, float* s, cudaStream_t stream);

/* ---- W8A8 row-wise-scaled GEMMs (tensor-core bound) ---------------------------------------- */
/* Kernel choice of the GEMM entries below and of rh3_conv3d_causal (no reference counterpart): 0 = one CTA per tile, 1 (the
 * default) = CTA pairs (clusters of two, tcgen05 cta_group::2): 256 x 256 GEMM tiles with each CTA loading its own half of
 * B, for calls with more than 128 rows and columns; two site tiles of the convolution per pair with each CTA loading half of
 * the weight rows, for calls with more than one site tile. Returns the previous setting; process-wide. Results are the same
 * bits either way. */
int rh3_gemm_use_pairs(int on);
/* out[M,N] bf16 = ((acc * xs[m]) * ws[n]) + bias[n]; xq[M,K] (row stride lda), wq[N,K] contiguous.
 * bias may be NULL. acc_dump (optional, [M,N] int32 / fp32 bits) receives the raw accumulators.
 * Replaces int8_rowwise_gemm / fp8_rowwise_gemm (custom_nodes/rapid_h3/csrc/fp8_rowwise.cu:512-584)
 * and the emulation in kernels.linear (kernels.py:129-137). */
int rh3_gemm_w8a8(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws, const void* bias,
                  int64_t M, int64_t N, int64_t K, int kind, void* out, int64_t ldo, int32_t* acc_dump,
                  cudaStream_t stream);
/* resid[M,N] = bf16(fma(bf16((acc*xs)*ws), gate[n], resid)) in place (row stride ldr). M == 0 is a no-op.
 * Replaces int8_gemm_gated_residual (fp8_rowwise.cu:333-389, :587-608). */
int rh3_gemm_w8a8_gated_residual(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                                 const void* gate, void* resid, int64_t ldr, int64_t M, int64_t N, int64_t K,
                                 int kind, cudaStream_t stream);
/* wq rows interleaved [g 4j..4j+3 | u 4j..4j+3]; out[M, N/2] = bf16(silu(bf16 g) * bf16 u).
 * Replaces int8_gemm_swiglu (fp8_rowwise.cu:29-107, :611-629; row order cutlass_fp8.py:55-62). */
int rh3_gemm_w8a8_swiglu(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws, int64_t M,
                         int64_t N, int64_t K, int kind, void* out, int64_t ldo, cudaStream_t stream);

/* ---- attention pre-pass (HBM-bound) and INT8 flash attention (tensor-core bound) ----------- */
/* y = per-(token, head) RMSNorm over 128 channels (weight bf16[128]) followed, when rope_table is
 * not NULL, by the split-half partial 3-D RoPE: rot_dim 96, pairs (i, i+48), table bf16 [S,48,2,2] =
 * (cos, -sin, sin, cos); channels 96..127 are normalised only. x, y: [S, H, 128] views with element
 * strides (token, head); y may alias x. Replaces comfy-kitchen's rms_rope_split_half_ as restated in
 * custom_nodes/rapid_h3/csrc/attn_int8.cu:217-260 (rms_rope_row) / :382-399 (rms_rope_only), with IEEE
 * division and square root instead of the .approx forms. */
int rh3_rmsnorm_rope3d(const void* x, int64_t x_ss, int64_t x_sh, void* y, int64_t y_ss, int64_t y_sh, int64_t S,
                       int64_t H, const void* weight, float eps, const void* rope_table, cudaStream_t stream);
/* Bytes of scratch rh3_attn_kv_stats needs for L tokens and H heads (returns the size, not a status). */
int64_t rh3_attn_kv_stats_scratch_bytes(int64_t L, int64_t H);
/* kmean, vmean, vscale: fp32 [H,128]. Per-(head, channel) mean of K and V over the L tokens (sums in
 * 256-token chunks: 16 groups of 16 tokens, tokens, groups and chunks each in order) and
 * vscale = max(max|v - vmean|, 1e-8) / 448. Rows 16-byte aligned.
 * Replaces stats_partial + stats_final (attn_int8.cu:82-109). */
int rh3_attn_kv_stats(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t L,
                      int64_t H, void* scratch, int64_t scratch_bytes, float* kmean, float* vmean, float* vscale,
                      cudaStream_t stream);
/* Same result as rh3_attn_kv_stats, for callers that are not able to allocate device memory (a host
 * framework that owns all VRAM, a serving loop where cudaMalloc is forbidden, a plugin that only receives its
 * input and output buffers). The chunk partials go to a 16 MiB array built into the library image (held on
 * every GPU that loads the library until the process exits), so no scratch is passed and nothing is
 * allocated or freed. Limit: H * ceil(L/256) <= 8192; larger problems are rejected with an error.
 * The first call on a device looks up the array's device address; make that first call outside any stream
 * capture. All calls share the one array: two calls whose kernels overlap on the GPU (different streams)
 * race on it; calls on one stream are safe, and nothing needs to be cleared between calls. Host threads may
 * make their first calls concurrently (the address look-up is idempotent and stored atomically).
 * This entry point has no counterpart in the reference. */
int rh3_attn_kv_stats_noalloc(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh,
                              int64_t L, int64_t H, float* kmean, float* vmean, float* vscale, cudaStream_t stream);
/* codes int8 [H, Lpad, 128], scales fp32 [H, Lpad/64]: one abs-max scale per 64-token block per head,
 * s = max(amax, 1e-8)/127, q = clamp(rint((x - mean)/s), +-127); mean (fp32 [H,128]) may be NULL (Q).
 * Rows L..Lpad are written as zeros. Replaces quant_qk / quant_k_block (attn_int8.cu:130-170, :404-443)
 * with the per-64-block scales of bench/attn_emulate.py:88 (`q8(k - km, 1, 64)`). */
int rh3_attn_quant_qk(const void* x, int64_t x_ss, int64_t x_sh, int64_t L, int64_t Lpad, int64_t H,
                      const float* mean, void* codes, float* scales, cudaStream_t stream);
/* vt e4m3 [H, 128, Lpad] = e4m3((v - vmean) / vscale), transposed so keys are contiguous; columns
 * L..Lpad are zeros. Replaces quant_v's e4m3 branch (attn_int8.cu:452-496) with the per-channel
 * scale of bench/attn_emulate.py:16-18,101 (`f8(v - vm, 0)`). */
int rh3_attn_quant_v(const void* v, int64_t v_ss, int64_t v_sh, int64_t L, int64_t Lpad, int64_t H,
                     const float* vmean, const float* vscale, void* vt, cudaStream_t stream);
/* The whole pre-pass of one attention call in three launches (what the reference's `prepass`, attn_int8.cu:2568-2644,
 * does in five, incl. its `_rr` forms that fuse the q/k RMSNorm + RoPE, :297-340 / :360-399):
 *   q [Lq,H,128], k, v [Lk,H,128] bf16 views (element strides given; rows 16-byte aligned).
 *   q_weight / k_weight (bf16 [128], both or neither): when given, q and k are raw and get the per-head RMSNorm (eps)
 *   and, with rope_table (bf16 [L,48,2,2], needs Lq == Lk), the 3-D RoPE of rh3_rmsnorm_rope3d first. The normalised k
 *   is written to k_roped (strides kr_ss, kr_sh; it may be k itself) because the K quantizer needs the mean of the
 *   whole sequence before it can run; the normalised q is quantized from registers and only stored when q_roped is
 *   not NULL. scratch: rh3_attn_kv_stats_scratch_bytes(Lk, H) bytes.
 *   Outputs as rh3_attn_quant_qk / rh3_attn_quant_v / rh3_attn_kv_stats define them: q8 [H,Lq_pad,128], qs [H,Lq_pad/64],
 *   k8 [H,Lk_pad,128], ks [H,Lk_pad/64], vt [H,128,Lk_pad], vscale, vmean, kmean [H,128]. Lq_pad % 256 == 0,
 *   Lk_pad % 128 == 0. */
int rh3_attn_prepass(const void* q, int64_t q_ss, int64_t q_sh, int64_t Lq, int64_t Lq_pad, const void* k, int64_t k_ss,
                     int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t Lk, int64_t Lk_pad, int64_t H,
                     const void* q_weight, const void* k_weight, float eps, const void* rope_table, void* q_roped,
                     int64_t qr_ss, int64_t qr_sh, void* k_roped, int64_t kr_ss, int64_t kr_sh, void* scratch,
                     int64_t scratch_bytes, void* q8, float* qs, void* k8, float* ks, void* vt, float* vscale,
                     float* vmean, float* kmean, cudaStream_t stream);
/* ---- token-scaled attention: the numerics of the reference's production attention ("config 80" family incl.
 * 90 / 94 / 190 / 194: custom_nodes/rapid_h3/csrc/README.md "What it computes", csrc/attn_cake/DESIGN.md section 2,
 * dispatch attn_int8.cu:2568-2644, kernels cake/attn_cake.cuh:113-491) ---- */
/* Pre-pass (five launches), arguments as rh3_attn_prepass except:
 *   q8 [H,Lq_pad,128], k8 [H,Lk_pad,128]: int8 codes of the 128-point Hadamard rotation of q and of k - kmean,
 *   ONE SCALE PER TOKEN: qs [H,Lq_pad]; ksb [H,Lk_pad/128,2,128] = per key tile 128 multipliers (key scale / 128:
 *   the unnormalised rotation multiplies Q.K^T by 128) followed by 128 biases (0; -inf for the padding keys);
 *   vt [H,128,Lk_pad] = int8((v - vmean) / vscale) with vscale = max|v - vmean| / 127 per channel. */
int rh3_attn_tok_prepass(const void* q, int64_t q_ss, int64_t q_sh, int64_t Lq, int64_t Lq_pad, const void* k,
                         int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t Lk,
                         int64_t Lk_pad, int64_t H, const void* q_weight, const void* k_weight, float eps,
                         const void* rope_table, void* q_roped, int64_t qr_ss, int64_t qr_sh, void* k_roped,
                         int64_t kr_ss, int64_t kr_sh, void* scratch, int64_t scratch_bytes, void* q8, float* qs,
                         void* k8, float* ksb, void* vt, float* vscale, float* vmean, float* kmean,
                         cudaStream_t stream);
/* Main kernel on those operands: int8 Q.K^T into int32, t_j = s * ksb scale + ksb bias, P = u8 against each key
 * tile's own row maximum, u8 x s8 P.V into int32 per tile, folded into the fp32 output with
 * ts = 2^(tile max - running max); row sums from the quantized P; out = (O/l) * vscale + vmean, bf16
 * [Lq, H, 128] (element strides o_ss, o_sh). */
int rh3_attn_int8_tok(const void* q8, const float* qs, const void* k8, const float* ksb, const void* vt,
                      const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk, int64_t Lk_pad,
                      int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh, cudaStream_t stream);
/* out[Lq, H, 128] bf16 (element strides o_ss, o_sh) = softmax(Q.K^T * softmax_scale) . V from the
 * pre-pass operands: int8 Q.K^T into int32, base-2 online softmax in fp32, P as e4m3 against the
 * running maximum, e4m3 P.V into fp32, out = (O/l) * vscale + vmean. Lq may differ from Lk.
 * Lq_pad (the padded row count of q8 / qs per head) must be a multiple of 256, Lk_pad a multiple of 128.
 * Replaces attention_impl / the attn_fwd5 FP8-P.V kernel (attn_int8.cu:1538-1759, :2749-2849). */
int rh3_attn_int8(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                  const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk, int64_t Lk_pad,
                  int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh, cudaStream_t stream);
/* rh3_attn_int8, and in addition the exact int32 scores Q8 . K8^T of one 128 x 128 tile (query tile q_tile, key
 * tile kv_tile, of `head`) are written to s_dump [128][128] int32 (device memory): the accumulator the softmax
 * reads, for bit-exact checks against an integer matrix product. A verification hook in the spirit of the
 * reference's ext().int8_prepass (attn_int8.cu:2692-2704); the reference has no dump of the scores themselves. */
int rh3_attn_int8_dump_scores(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                              const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                              int64_t Lk_pad, int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh,
                              int64_t head, int64_t q_tile, int64_t kv_tile, int32_t* s_dump, cudaStream_t stream);

/* ---- VAE decoder: causal 3-D convolution as implicit GEMM, GroupNorm + SiLU, upsampling --------------- */
/* None of these has a counterpart in the reference (its VAE fast path accelerates a transformer decoder,
 * custom_nodes/rapid_h3/vae_fast.py:430-437); they implement the causal conv3d decoder of the benchmark
 * configuration. Activations are channels-last bf16 [N, T, H, W, C]. */
/* out = bf16(conv3x3x3(x, w) + bias (+ residual)); w is [Cout, 27, Cin] with tap = (dt*3 + dh)*3 + dw; zero
 * padding of one pixel in H and W and of two frames before t = 0 (causal). Cin % 64 == 0, Cout % 16 == 0.
 * bias, residual and gn_part may be NULL. gn_part (fp32 [rh3_conv3d_gn_part_rows(), 32, 2]) receives
 * per-row-block partial (sum, sum of squares) of the stored outputs for each of 32 GroupNorm groups.
 * halo_frames = 2: x holds T + 2 frames per sample, the first two being the frames that precede output frame 0
 * (the previous time shard's last frames) in place of the causal zero padding; out, residual and the statistics
 * still cover T frames. halo_frames = 0: plain causal padding. */
int rh3_conv3d_causal(const void* x, const void* w, const void* bias, const void* residual, void* out,
                      float* gn_part, int64_t N, int64_t T, int64_t H, int64_t W, int64_t Cin, int64_t Cout,
                      int64_t halo_frames, cudaStream_t stream);
/* Number of row blocks (first dimension of gn_part) for an output of N x T x H x W sites (a size, not a status). */
int64_t rh3_conv3d_gn_part_rows(int64_t N, int64_t T, int64_t H, int64_t W);
/* sums (fp64 [N, 32, 2]) = per-sample, per-group (sum, sum of squares) over rows_per_sample row blocks. */
int rh3_gn_reduce(const float* gn_part, int64_t rows_per_sample, int64_t N, double* sums, cudaStream_t stream);
/* y = silu((x - mean[n, g]) * rstd[n, g] * gamma[c] + beta[c]); mean_rstd is fp32 [N, 32, 2]; 32 groups. */
int rh3_gn_silu_apply(const void* x, const float* mean_rstd, const void* gamma, const void* beta, int64_t N,
                      int64_t sites_per_sample, int64_t C, void* y, cudaStream_t stream);
/* y[N, 2T-1, 2H, 2W, C]: nearest-neighbour 2x in space, causal 2x in time (the first frame is not repeated). */
int rh3_upsample_causal2x(const void* x, void* y, int64_t N, int64_t T, int64_t H, int64_t W, int64_t C,
                          cudaStream_t stream);
/* Depth-to-space by 8 of the decoder head: y [N, T, H, W, 192] (channel = (ch*8 + dy)*8 + dx) -> rgb [N, 3, T, 8H, 8W]. */
int rh3_depth_to_space8(const void* y, void* rgb, int64_t N, int64_t T, int64_t H, int64_t W, cudaStream_t stream);

/* Second int8 pass of the text encoder's `int8_rot` linears on its outlier rows: for i < n and r = rows[i],
 * q2[i], s2[i] = int8 row quantizer of rotate(x[r]) - q1[r] * s1[r]  (x fp32 [*, K], q1 / s1 the first pass's codes and
 * scales). Replaces the torch expression of te_quant._TELinear.__call__ (custom_nodes/rapid_h3/te_quant.py:96-105). */
int rh3_rot_residual_quant_rows_i8(const float* x, int64_t ldx, const void* q1, int64_t ldq1, const float* s1,
                                   const int32_t* rows, int64_t n, int64_t K, void* q2, float* s2, cudaStream_t stream);

/* ---- sequence parallelism: the two exchanges of Ulysses attention done by the kernels themselves ----
 * No reference counterpart (the reference is single-GPU). Both write with plain stores into buffers that may be
 * on peer GPUs (pointers obtained by the host through CUDA IPC / symmetric memory); neither waits on a peer:
 * the caller orders producers and consumers with a stream-ordered barrier (e.g. a one-element all-reduce).
 * rh3_rope_scatter_heads: RMSNorm + 3-D RoPE of q and k (as rh3_rmsnorm_rope3d) of this rank's S tokens, rows
 *   [S, 3*H*128] = q | k | v; head h goes to dst[h / (H/P)], laid out [total tokens, 3, (H/P)*128], at token
 *   row0 + s. v is copied unchanged.
 * rh3_attn_int8_scatter: rh3_attn_int8 whose output rows [dst_start[r], dst_start[r+1]) are stored to
 *   dst[r] + (row - dst_start[r]) * o_ss + head * o_sh (1 <= n_dst <= 8, dst_start[0] = 0, dst_start[n_dst] >= Lq). */
int rh3_rope_scatter_heads(const void* qkv, int64_t ld, int64_t S, int64_t H, int64_t P, int64_t row0,
                           const void* q_weight, const void* k_weight, float eps, const void* rope_table,
                           void* const* dst, cudaStream_t stream);
int rh3_attn_int8_scatter(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                          const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                          int64_t Lk_pad, int64_t H, float softmax_scale, void* const* dst, const int64_t* dst_start,
                          int64_t n_dst, int64_t o_ss, int64_t o_sh, cudaStream_t stream);

/* ---- fp16 ops of the VAE transformer decoder (the callers of the int8 path at fp16 activations) ----
 * rh3_vae_out_quant: o [B, H, S, D] fp16 head-major attention output -> q int8 [B*S, H*D], scales fp32 [B*S]:
 *   nan_to_num on load, H256 rotation in comfy-kitchen's stage order, int8 with value / scale / quotient rounded
 *   through fp16. Replaces vae_ops.vae_out_quant (custom_nodes/rapid_h3/csrc/vae_ops.cu:63-142,366-385).
 * rh3_vae_gemm: out fp16 [M, N] = fp16(fp16((acc * xs[m]) * ws[n] + bias[n]) * rscale[n] + resid[m, n]) when a
 *   residual is given, else fp16((acc * xs[m]) * ws[n] + bias[n]). Replaces vae_ops.vae_gemm
 *   (vae_ops.cu:150-227,387-403; called from vae_fast._linear, vae_fast.py:118-169).
 * rh3_vae_gemm_swiglu: weight rows interleaved [g 4j..4j+3 | u 4j..4j+3]; g, u = fp16((acc*xs)*ws + bias),
 *   out fp16 [M, N/2] = fp16(g / (1 + e^-g) * u). Replaces vae_ops.vae_gemm_swiglu (vae_ops.cu:228-345,405-420). */
int rh3_vae_out_quant(const void* o_f16, int64_t B, int64_t H, int64_t S, int64_t D, void* q, float* scales,
                      cudaStream_t stream);
/* rh3_vae_quant_rows: the row arithmetic of rh3_vae_out_quant on a row-major fp16 matrix x [M, K] (the plain
 * activation case of the quantizer the decoder's linears run on their inputs, vae_fast._quantize,
 * custom_nodes/rapid_h3/vae_fast.py:71-85). */
int rh3_vae_quant_rows(const void* x_f16, int64_t ldx, int64_t M, int64_t K, void* q, float* scales,
                       cudaStream_t stream);
/* The same quantizer with the fused activation prologue of vae_fast._quantize's `act` argument (vae_fast.py:71-85):
 * act 1 = "rms_norm": x [M, K], y = (x / sqrt(mean(x^2) + eps)) * act_weight (fp16 [K], may be NULL);
 * act 2 = "swiglu": x [M, 2K] = [gate | up], y = gate / (1 + e^-gate) * up. y is kept in fp32 into the rotation. */
int rh3_vae_quant_rows_act(const void* x_f16, int64_t ldx, int64_t M, int64_t K, int act, const void* act_weight_f16,
                           float eps, void* q, float* scales, cudaStream_t stream);
int rh3_vae_gemm(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws, const void* bias_f16,
                 const void* rscale_f16, const void* resid_f16, int64_t ldr, int64_t M, int64_t N, int64_t K,
                 void* out_f16, int64_t ldo, cudaStream_t stream);
int rh3_vae_gemm_swiglu(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                        const void* bias_f16, int64_t M, int64_t N, int64_t K, void* out_f16, int64_t ldo,
                        cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RAPIDH3_B200_H_ */
