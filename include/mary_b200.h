/* mary_b200.h -- C ABI of the B200 (sm_100a) kernels behind maryml's quantized
 * inference op surface.
 *
 * Every entry point takes plain device pointers, sizes and scalars, enqueues its
 * work on the given CUDA stream and returns without synchronising (the one
 * exception, the weight quantizer's amax readback, is the reference's own).
 * Outputs and workspaces are allocated by the caller, so a Rust wrapper can hand
 * out buffers of its own arena and keep ownership. Return value: 0, or a negative
 * MB_ERR_* code with the text available from mb_last_error(). Preflight refusals
 * (shape, alignment, extent) happen before any launch, as in the reference.
 *
 * Each declaration cites the reference interface it replaces (file:line, paths
 * relative to the reference project root).
 *
 * Layouts
 *   codes      [rows, K/2] bytes, E2M1, the lower K index in the LOW nibble
 *   scales     [rows, K/16] E4M3 bytes, row-major             (MB_SF_ROWMAJOR)
 *   scales     tiled for the tensor-core GEMM                 (MB_SF_TILED):
 *              512-byte atoms of 128 rows x 4 scales, byte (row%32)*16 +
 *              (row/32%4)*4 + kb%4 inside an atom, atoms ordered [row/128][kb/4],
 *              K padded to a multiple of 256 elements, rows to 128
 *   scale2     one f32 per tensor (per expert in a bank)
 */
#ifndef MARY_B200_H
#define MARY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mb_ctx mb_ctx;
typedef void* mb_stream; /* a cudaStream_t */

enum {
  MB_OK = 0,
  MB_ERR_INVALID = -1, /* refused before launch: shape, alignment, extent, non-finite scale */
  MB_ERR_CUDA = -2,    /* a CUDA runtime/driver call failed */
  MB_ERR_NONFINITE = -3, /* the reference refuses a weight holding NaN/Inf */
  MB_ERR_DEVICE_FLAG = -4, /* a kernel raised a status word (timeout, bad routing) */
  MB_ERR_UNAVAILABLE = -5  /* an optional dependency (NCCL) could not be loaded */
};

enum { MB_DT_BF16 = 0, MB_DT_F32 = 1 };
enum { MB_SF_ROWMAJOR = 0, MB_SF_TILED = 1 };

/* Activation quantizer recipes. */
enum {
  /* quantize_block with a second-level scale `input_scale`: block byte =
   * e4m3(min((amax/6)/input_scale, 448)), codes = cvt(x / (f32(byte)*input_scale)).
   * src/nn/nvfp4_gemv.rs:140-172, used by src/nn/nvfp4_gemm.rs:644-669. */
  MB_QUANT_SCALED = 0,
  /* no second level, hoisted reciprocal: byte = e4m3(min(amax/6, 448)),
   * codes = cvt(x * fl(1/f32(byte))). src/models/inkling/fp4quant.rs:199-238. */
  MB_QUANT_RECIP = 1,
  /* per-row second-level scale amax_row/2688 written to `rowscale`.
   * src/nn/nvfp4_gemm.rs:757-813. */
  MB_QUANT_ROWS = 2
};

/* GEMM epilogues. */
enum {
  MB_EPI_PLAIN = 0,            /* out = acc * alpha [* rowscale[m]] */
  MB_EPI_SWIGLU_INTERLEAVED = 1,/* columns (2i, 2i+1) = (gate, up), each rounded to bf16, then
                                  out[m, i] = bf16(silu(gate) * up); out has N/2 columns.
                                  src/models/inkling/fp4gemm.rs:472-507 fused into the GEMM. */
  MB_EPI_SWIGLU_ROUNDED = 3,    /* the same with silu(gate) itself rounded to bf16 before the product and
                                  exact exp/divide: the rounding points of the dense layer's swiglu on
                                  bf16 gate and up tensors (mb_swiglu), so the fusion changes no bit. */
  /* flags for the two SwiGLU epilogues: the bf16 result is not stored but quantized where it is
   * produced (32 accumulator columns = 16 results = one NVFP4 block): `out` receives the code
   * plane [m, n/4 bytes] and `out_sf` the tiled scale plane of an [m, n/2] tensor, the bytes
   * mb_nvfp4_quantize_act would have written for the stored bf16 result. */
  MB_EPI_QUANT_RECIP = 0x100,   /* recipe MB_QUANT_RECIP */
  MB_EPI_QUANT_SCALED = 0x200   /* recipe MB_QUANT_SCALED with input_scale 1 */
};

/* ---- context ---------------------------------------------------------------- */
/* Replaces the cubecl ComputeClient the reference's launch functions take
 * (src/models/inkling/rawcuda.rs:31-80). One per device and host thread. */
int mb_ctx_create(int device, mb_ctx** out);
void mb_ctx_destroy(mb_ctx* ctx);
/* The persistent GEMM kernels launch one CTA (or CTA pair) per SM and walk their tiles in a fixed
 * round-robin; a collective that runs beside them on another stream (the all-reduce of the previous
 * chunk of a prompt, src/models/inkling/tpcomm.rs:1453-1467) holds some SMs for its whole duration and
 * would stall the CTAs that were to run there. `sms` > 0 makes those kernels use at most that many SMs,
 * 0 restores all of them. No counterpart in the reference, whose GEMMs are not persistent. */
int mb_ctx_set_sm_limit(mb_ctx* ctx, int sms);
/* Wall-time budget of one wait on a peer rank inside the fused exchange kernels (mb_tp_reduce_residual):
 * 100 us .. 60 s, one second by default. A wait that runs out ends the kernel with status word 0 set to
 * the wait's code (51: a peer's partials, 52: a peer's slice), word 3 the microseconds waited and word 4
 * the rank waited for; mb_check_flags then returns MB_ERR_DEVICE_FLAG and the context stays usable. The
 * reference bounds its collectives by a watchdog on the host (src/models/inkling/tpcomm.rs:10-38). */
int mb_ctx_set_wait_limit_us(mb_ctx* ctx, uint32_t microseconds);
const char* mb_last_error(mb_ctx* ctx);
const char* mb_version(void);
/* Reads and clears the device status words (bounded-wait timeouts, non-finite
 * router logits, bad routing plans); synchronises `stream`. The reference reads
 * such flags later on the host: src/models/inkling/routetopk.rs:39-45,
 * src/models/inkling/devplan.rs:248-300. Returns MB_ERR_DEVICE_FLAG if any is set. */
int mb_check_flags(mb_ctx* ctx, mb_stream stream, int32_t* flags_out8);

/* ---- NVFP4 codec ---------------------------------------------------------------- */
/* Nvfp4::quantize (src/nn/nvfp4_gemv.rs:284-351): amax over the tensor (one host
 * round trip), scale2 = amax/(6*448) or 1.0, then one 16-block per thread.
 * w: [n, k] bf16 contiguous, k % 32 == 0. Writes row-major codes and scales.
 * Synchronises `stream` once. MB_ERR_NONFINITE for a NaN/Inf weight. */
int mb_nvfp4_quantize_weight(mb_ctx* ctx, mb_stream stream, const void* w_bf16, size_t n, size_t k,
                             uint8_t* codes, uint8_t* scales, float* scale2_host_out);

/* quantize_kernel / quantize_nvfp4(_bf16) / quantize_rows_kernel
 * (src/nn/nvfp4_gemv.rs:123-172, src/models/inkling/fp4quant.rs:199-238,
 * src/nn/nvfp4_gemm.rs:757-813). x: [rows, k] bf16 or f32, k % 16 == 0 (k % 64
 * for the tensor-core GEMM). sf_layout selects row-major or tiled scales; a tiled
 * plane must hold mb_nvfp4_sf_bytes(rows, k) bytes. rowscale: [rows] f32 output for
 * MB_QUANT_ROWS, else NULL. gather: optional [rows] int32 source-row map
 * (src/models/inkling/moegroup.rs:313-331: out row r reads x row gather[r]; a
 * negative entry is a zero row); src_rows = rows of x when gather is given. */
int mb_nvfp4_quantize_act(mb_ctx* ctx, mb_stream stream, const void* x, int x_dtype, size_t rows, size_t k,
                          int recipe, float input_scale, const int32_t* gather, size_t src_rows,
                          uint8_t* codes, uint8_t* scales, int sf_layout, float* rowscale);

/* gather_rows(_bf16) followed by the activation quantizer (src/models/inkling/moegroup.rs:313-331,
 * :3429-3470) with the two steps exchanged: a row's NVFP4 bytes do not depend on where the row
 * lands, so the tokens are quantized once ([src_rows, k], tiled scales) and their planes are
 * copied into plan order: out row r = source row gather[r]; a negative entry is a zero row
 * (zero codes, zero scales); an entry >= src_rows raises the plan flag and is written as zeros.
 * Both scale planes are tiled; the output planes hold `rows` rows. k % 64 == 0. */
int mb_nvfp4_gather_rows(mb_ctx* ctx, mb_stream stream, const uint8_t* codes, const uint8_t* sf_tiled,
                         size_t src_rows, size_t k, const int32_t* gather, size_t rows, uint8_t* out_codes,
                         uint8_t* out_sf_tiled);

/* transcode_to_nvfp4 (src/nn/mxfp4.rs:319-375): the exact relabelling of an MXFP4 tensor (E2M1
 * codes, one E8M0 scale per 32 values) as NVFP4. The codes are used as they are; this call only
 * re-expresses the scales: e8m0 [n] device bytes -> block_scales [2 n] E4M3 bytes, row-major (tile
 * them with mb_nvfp4_tile_scales for the GEMM), and the global scale 2^g with g = e_max - 8, a
 * power of two, returned on the host. Every decoded weight E2M1[code] * e4m3(scale) * 2^g equals
 * E2M1[code] * 2^(b - 127) bit for bit. MB_ERR_NONFINITE for a 0xFF scale (the first index is in
 * the message), MB_ERR_INVALID when the exponents span more than E4M3's 18 octaves or 2^g is not a
 * normal f32. Synchronises `stream` once. */
int mb_mxfp4_to_nvfp4_scales(mb_ctx* ctx, mb_stream stream, const uint8_t* e8m0, size_t n, uint8_t* block_scales,
                             float* global_scale_host_out, int* global_exp_host_out);

/* dequantize_nvfp4(_bf16) (src/models/inkling/fp4quant.rs:437-459) and
 * nvfp4::decode_payload (src/nvfp4.rs:170-182): out = E2M1[code]*(e4m3(scale)*scale2). */
int mb_nvfp4_dequantize(mb_ctx* ctx, mb_stream stream, const uint8_t* codes, const uint8_t* scales_rowmajor,
                        float scale2, size_t rows, size_t k, void* out, int out_dtype);

/* Size of a tiled scale plane, and the re-layout of a row-major plane into it.
 * The reference pre-permutes weights for its MMA the same way at load
 * (src/models/inkling/fp4gemm.rs:1279-1367); `upload` still takes the canonical planes. */
size_t mb_nvfp4_sf_bytes(size_t rows, size_t k);
int mb_nvfp4_tile_scales(mb_ctx* ctx, mb_stream stream, const uint8_t* scales_rowmajor, size_t rows, size_t k,
                         uint8_t* scales_tiled);
int mb_nvfp4_untile_scales(mb_ctx* ctx, mb_stream stream, const uint8_t* scales_tiled, size_t rows, size_t k,
                           uint8_t* scales_rowmajor);

/* ---- linears ---------------------------------------------------------------------- */
/* Nvfp4::gemv (src/nn/nvfp4_gemv.rs:202-250, 529-578): [rows<=8, k] x [n, k]^T,
 * W4A16: every product x * (w * block scale) is exact in f32 (the decoded, scaled weight has at most
 * 7 significant bits), sums carried in f32, x scale2 once, one cast. One to eight rows cost the same
 * (the rows are the N side of a warp-level tensor-core product over 16 weight rows).
 * x 16-byte aligned, k % 32 == 0. */
int mb_nvfp4_gemv_w4a16(mb_ctx* ctx, mb_stream stream, const void* x_bf16, size_t rows, const uint8_t* codes,
                        const uint8_t* scales_rowmajor, float scale2, size_t n, size_t k, void* out,
                        int out_dtype);

/* mb_nvfp4_gemv_w4a16 is one kernel: the bf16 rows are used as they are (a decoded weight goes from its f16 pattern
 * to bf16 by a three-bit shift and one packed multiply by scale * 2^112, exact), and a weight with few rows and a
 * long K is cut along K with the ranges of a 16-row block as the CTAs of one thread-block cluster: their sums meet in
 * distributed shared memory and are added in range order, so the result does not depend on timing and no workspace
 * is needed.
 * mb_nvfp4_gemv_w4a16_ws is the same call for weights of up to four 16-row blocks per SM; for taller ones, which
 * are bound by instruction issue, and given a workspace (mb_nvfp4_gemv_workspace bytes, 256-byte aligned), it takes
 * a two-kernel form (MB_GEMV_TWO_PASS=1 / 0 in the environment forces one form or the other): a pass of one
 * block per row makes an f16 copy of the rows (exact for zero, infinite, NaN and every value in f16's normal range;
 * a row with a finite value outside it raises a flag in the workspace and the call takes the bf16 form), the product
 * runs f16 x f16 (five instructions per four weights instead of eight) and K ranges meet in the workspace, the block
 * that arrives last adding them in range order. Every product is exact in f32 in both forms and the ranges are added
 * in the same order: the forms differ only where their range counts differ. */
size_t mb_nvfp4_gemv_workspace(size_t rows, size_t n, size_t k);
int mb_nvfp4_gemv_w4a16_ws(mb_ctx* ctx, mb_stream stream, const void* x_bf16, size_t rows, const uint8_t* codes,
                           const uint8_t* scales_rowmajor, float scale2, size_t n, size_t k, void* out, int out_dtype,
                           void* workspace, size_t workspace_bytes);

/* Nvfp4::project(W4a4) / project_w4a4_scaled / project_w4a4_rows and fp4_linear_launch
 * (src/nn/nvfp4_gemm.rs:200-291, 644-694, 814-945; src/models/inkling/fp4gemm.rs:154-245):
 * out[m, n] = (sum_k a[m,k] b[n,k]) * alpha [* rowscale[m]], both operands NVFP4
 * planes with TILED scales; tcgen05 block-scaled MMA, f32 accumulation in TMEM.
 * k % 64 == 0, n % 8 == 0. out: [m, n] bf16 or f32 ([m, n/2] bf16 for the SwiGLU epilogue). */
int mb_nvfp4_gemm_w4a4(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                       const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* rowscale, float alpha,
                       size_t m, size_t n, size_t k, void* out, int out_dtype, int epilogue);

/* The same product for decode-sized activations (m <= 128), where a [m, n] output has too few
 * tiles to keep 148 SMs streaming weights (the reference's own answer at this size is its
 * one-plane-per-tile grid, src/nn/nvfp4_gemm.rs:200-291): K is cut into slices whose sums are
 * added in slice order (deterministic) with the epilogue scale. Where the device holds every
 * tile's slices as one thread-block cluster (mb_gemm_splitk_plan below), they meet in
 * distributed shared memory inside the product's kernel and `workspace` is not touched;
 * otherwise they land in f32 planes of `workspace` and a second kernel adds them.
 * mb_nvfp4_gemm_splitk_workspace returns the bytes to provide for that case, 0 when the shape
 * is not split; with a null or short workspace the call is mb_nvfp4_gemm_w4a4 (which takes the
 * cluster form on its own where it applies). */
size_t mb_nvfp4_gemm_splitk_workspace(size_t m, size_t n, size_t k);
/* How such a product (operands 0: NVFP4 x NVFP4, 1: bf16 x bf16) runs on this context's device. With up to eight
 * slices the K slices of an output tile are the CTAs of one thread-block cluster and meet in distributed shared
 * memory inside the product's own kernel: no planes, no second kernel, no workspace needed, also through
 * mb_nvfp4_gemm_w4a4 / mb_bf16_gemm. *cluster_slices is that slice count (0: the form does not apply: more than
 * eight slices, or more tiles than clusters the device holds at once), *plane_slices the count of the plane form
 * (0 or 1: not split). The slices are added in slice order in both forms, so a call gives the same bits every time;
 * the two forms give the same bits whenever their slice counts agree. */
int mb_gemm_splitk_plan(mb_ctx* ctx, int operands, size_t m, size_t n, size_t k, int* cluster_slices, int* plane_slices);
int mb_nvfp4_gemm_w4a4_splitk(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                              const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* rowscale, float alpha,
                              size_t m, size_t n, size_t k, void* out, int out_dtype, void* workspace,
                              size_t workspace_bytes);

/* fp4_linear_grouped(_bf16)_launch (src/models/inkling/moegroup.rs:430-751): the
 * stacked rows of all active experts against an expert bank. a: [m_cap, k] planes
 * (each expert's rows padded to 128). bank: [experts, n, k] planes with tiled scales
 * per expert. tile_expert: [m_cap/128] int32, the expert of each 128-row tile or -1;
 * n_tiles_dev: device int32, tiles in use. alpha: [experts] f32 (the expert's scale2).
 * row_tok: optional [m_cap] int32, the plan's token of each stacked row; rows with a negative
 * entry are the padding that closes an expert's last tile, and with row_tok given a bf16 or f32
 * output keeps its old bytes there instead of receiving the products of zero rows (a third of
 * the rows at 4096 tokens x top-8 over 128 experts). Quantized output is always written whole. */
int mb_nvfp4_gemm_w4a4_grouped(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                               const uint8_t* bank_codes, const uint8_t* bank_sf_tiled, const float* alpha,
                               const int32_t* tile_expert, const int32_t* n_tiles_dev, size_t m_cap,
                               size_t experts, size_t n, size_t k, void* out, int out_dtype, int epilogue,
                               void* out_sf, const int32_t* row_tok);

/* w4a4_grouped_bf16 (src/nn/nvfp4_gemm.rs:462-523) with its two launches as two entry points: the decode-time
 * grouped experts, one activation row per group against expert ids[g] of a bank (GroupedBank, :438-451).
 * mb_nvfp4_quantize_grouped = quantize_grouped_kernel (:293-313): x is one shared bf16 row [k]
 * (x_per_group = 0) or one row per group [groups, k]; group g is quantized by the divide recipe with the
 * second-level scale input_scale[ids[g]] into codes [groups, k/2] and ROW-MAJOR scales [groups, k/16].
 * mb_nvfp4_gemv_w4a4_grouped = w4a4_grouped_kernel (:320-432): out[g, :] = (a[g, :] . bank[ids[g]]^T) *
 * alpha[ids[g]] with alpha the host's f32 scale2 * input_scale per expert; bank planes [experts, n, k/2] codes
 * and [experts, n, k/16] ROW-MAJOR scales, streamed once at HBM rate. Per group this is
 * Nvfp4::project_w4a4_scaled on one row up to the order of the f32 sums. ids: [groups] device int32,
 * ascending and distinct in the reference's use; an id outside the bank raises the plan flag of the context
 * (group + 1) and that group's row comes out as zeros. k % 64 == 0, n % 8 == 0, groups <= 65535. */
int mb_nvfp4_quantize_grouped(mb_ctx* ctx, mb_stream stream, const void* x_bf16, int x_per_group, const int32_t* ids,
                              size_t groups, const float* input_scale, size_t experts, size_t k, uint8_t* codes,
                              uint8_t* scales_rowmajor);
int mb_nvfp4_gemv_w4a4_grouped(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_scales_rowmajor,
                               const uint8_t* bank_codes, const uint8_t* bank_scales_rowmajor, const float* alpha,
                               const int32_t* ids, size_t groups, size_t experts, size_t n, size_t k, void* out,
                               int out_dtype);

/* Several projections of one input stacked along n (q|k|v, or gate and up interleaved row by
 * row), each stored tensor keeping its own global scale: colscale[n] holds the scale2 of the
 * tensor a column belongs to, out[m, c] = acc * colscale[c], rounded once, which is what the
 * separate products give (src/nn/nvfp4_gemm.rs:644-694 called once per projection). The
 * activation planes carry a unit global. epilogue: any MB_EPI_* word; out_sf as for the flags
 * above, else null. workspace: optional split-K planes as for mb_nvfp4_gemm_w4a4_splitk (plain
 * epilogue only). n % 32 == 0. */
int mb_nvfp4_gemm_w4a4_stacked(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                               const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* colscale, size_t m,
                               size_t n, size_t k, void* out, int out_dtype, int epilogue, void* out_sf,
                               void* workspace, size_t workspace_bytes);

/* bf16_linear_launch (src/models/inkling/bf16gemm.rs:64-152): [m, k] x [n, k]^T,
 * bf16 operands, f32 accumulation (tcgen05 kind::f16), out = acc * alpha as bf16 or
 * f32. k % 8 == 0. alpha carries the weight's scale2 when b is a decoded NVFP4 plane
 * (the W4A16 lane, src/nn/nvfp4_gemm.rs:93-197: scale2 applied once to the accumulator). */
int mb_bf16_gemm(mb_ctx* ctx, mb_stream stream, const void* a_bf16, const void* b_bf16, float alpha, size_t m,
                 size_t n, size_t k, void* out, int out_dtype);
/* Nvfp4::project(W4a16) / w4a16_linear_launch (src/nn/nvfp4_gemm.rs:93-197, src/models/inkling/w4a16gemm.rs):
 * [m, k] bf16 x [n, k]^T NVFP4 with the weight left four bits in HBM and no 16-bit copy of it anywhere: code
 * bytes arrive in shared memory by TMA, converter warps expand code x block scale to f16 (exact) into the
 * tensor core's operand tile, tcgen05 kind::f16 (bf16 A, f16 B) accumulates in f32, scale2 is applied once to
 * the accumulator, one cast. codes [n, k/2], scales [n, k/16] ROW-MAJOR (the canonical planes). k % 64 == 0,
 * n % 8 == 0. workspace: optional K-slice planes for products with few output tiles
 * (mb_nvfp4_gemm_w4a16_workspace bytes, 0 = never split; a null or short workspace runs unsplit). */
size_t mb_nvfp4_gemm_w4a16_workspace(size_t m, size_t n, size_t k);
int mb_nvfp4_gemm_w4a16(mb_ctx* ctx, mb_stream stream, const void* x_bf16, const uint8_t* codes,
                        const uint8_t* scales_rowmajor, float scale2, size_t m, size_t n, size_t k, void* out,
                        int out_dtype, void* workspace, size_t workspace_bytes);
/* The same product when the output has few tiles and K is long (the router projection
 * src/models/k3/router.rs:300-340 `Router::logits`: [tokens, hidden] x [experts, hidden]^T): K slices into f32 planes of
 * `workspace`, summed in slice order. mb_bf16_gemm_splitk_workspace gives the bytes, 0 = not split. */
size_t mb_bf16_gemm_splitk_workspace(size_t m, size_t n, size_t k);
int mb_bf16_gemm_splitk(mb_ctx* ctx, mb_stream stream, const void* a_bf16, const void* b_bf16, float alpha, size_t m,
                        size_t n, size_t k, void* out, int out_dtype, void* workspace, size_t workspace_bytes);

/* ---- MoE routing and permutation -------------------------------------------------- */
/* Router::scores/select/combine_weights/normalize, softmax branch
 * (src/models/k3/router.rs:343-471; device form src/models/inkling/routetopk.rs:112-217):
 * softmax over n_experts logits (f64 exp, f32 store), top-k by descending score with
 * ties to the lower index, weights renormalised w/(sum+1e-20)*scaling.
 * logits [tokens, n_experts] f32 -> idx [tokens, k] int32, weight [tokens, k] f32.
 * A non-finite logit raises the router flag of the context. n_experts <= 1024, k <= 32. */
int mb_router_topk_softmax(mb_ctx* ctx, mb_stream stream, const float* logits, size_t tokens, size_t n_experts,
                           size_t k, int renormalize, float scaling, int32_t* idx, float* weight);

/* The same route with the activation chosen and the selection bias of the `noaux_tc` gate
 * (src/models/k3/router.rs:343-446, RouterActivation::{Sigmoid, Softmax} and
 * Router::scores_for_choice): sigmoid scores are f32(1 / (1 + exp(-f64(x)))) per expert;
 * `bias` ([n_experts] f32, or NULL) is added to the scores for the SELECTION only, the
 * weights are gathered from the unbiased scores. A non-finite logit or biased score
 * raises the router flag. */
enum { MB_ROUTER_SOFTMAX = 0, MB_ROUTER_SIGMOID = 1 };
int mb_router_topk(mb_ctx* ctx, mb_stream stream, const float* logits, const float* bias, int activation,
                   size_t tokens, size_t n_experts, size_t k, int renormalize, float scaling, int32_t* idx,
                   float* weight);

/* The Inkling router decision with shared-expert sinks: router_topk_launch
 * (src/models/inkling/routetopk.rs:112-266) and its host twin route_from_logits
 * (src/models/inkling/block.rs:176-258). logits [tokens, n_routed + n_shared] f32. The k experts
 * are picked among the n_routed by sigmoid(logit) + bias[e] (f32; descending, ties to the lower
 * index); the bias takes no part in the weights. The k chosen logits followed by the n_shared sink
 * logits share one softmax over log_sigmoid (summed in that order):
 * weight = exp(lp - lse) * route_scale * global_scale -> weight [tokens, k] for the chosen experts,
 * shared_gammas [tokens, n_shared] for the sinks (NULL when n_shared == 0). The reference packs ids,
 * weights and a flag column into one f32 buffer for a single readback; here they are separate arrays
 * and a non-finite logit raises the router flag of the context (token + 1). n_routed % 32 == 0,
 * n_routed <= 512, n_shared <= 32, k <= 32. */
int mb_router_topk_sinks(mb_ctx* ctx, mb_stream stream, const float* logits, const float* bias, float global_scale,
                         float route_scale, size_t tokens, size_t n_routed, size_t n_shared, size_t k, int32_t* idx,
                         float* weight, float* shared_gammas);

/* RowPlan::build / plan_from_topk (src/models/inkling/moegroup.rs:1850-1909,
 * src/models/inkling/devplan.rs:216-301), on the device for any token count:
 * rows stacked expert-ascending then token-ascending, each expert padded to 128
 * rows. Outputs: row_tok [m_cap] (-1 = pad), row_wgt [m_cap], tok_rows [tokens, k]
 * (each token's rows, ascending), expert_rows [n_experts] counts, expert_row0
 * [n_experts] first stacked row, tile_expert [m_cap/128], n_tiles (1 int32).
 * m_cap = mb_moe_plan_rows(tokens, k, n_experts). workspace: mb_moe_plan_workspace bytes. */
size_t mb_moe_plan_rows(size_t tokens, size_t k, size_t n_experts);
size_t mb_moe_plan_workspace(size_t tokens, size_t k, size_t n_experts);
int mb_moe_plan(mb_ctx* ctx, mb_stream stream, const int32_t* idx, const float* weight, size_t tokens, size_t k,
                size_t n_experts, int32_t* row_tok, float* row_wgt, int32_t* tok_rows, int32_t* expert_rows,
                int32_t* expert_row0, int32_t* tile_expert, int32_t* n_tiles, void* workspace,
                size_t workspace_bytes);

/* scatter_weighted(_bf16) (src/models/inkling/moegroup.rs:1690-1716): out[t, :] =
 * sum over t's k rows, ascending, of fma(y[r, :], row_wgt[r], sum). y bf16 or f32. */
int mb_moe_scatter_weighted(mb_ctx* ctx, mb_stream stream, const void* y, int y_dtype, const float* row_wgt,
                            const int32_t* tok_rows, size_t tokens, size_t k, size_t h, float* out);

/* ---- attention ---------------------------------------------------------------------- */
/* flash_attention_launch (src/models/inkling/flash.rs:1140-1316) for the plain GQA
 * case (no window, no relative bias, no eviction gaps): softmax(scale*QK^T + causal)V.
 * q [batch, nq, heads*D] bf16, k/v [batch, keys, kv_heads*D] bf16 token-major,
 * out [batch, nq, heads*D] bf16. Query i of a sequence sits at absolute position
 * q0+i, key j at j; causal masks j > q0+i. D == 128. Decode (nq small) splits the
 * key axis and combines partial (o, m, l) exactly as flash.rs:892-966; workspace
 * from mb_attention_workspace(). */
size_t mb_attention_workspace(size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d);
int mb_attention(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v, size_t batch,
                 size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                 int causal, void* out, void* workspace, size_t workspace_bytes);
/* The same with a sliding window (banded_attention_kernel src/models/inkling/banded.rs:109-245 and the window
 * term of flash.rs:751-785): the query at position q sees the keys in (q - window, q]. Causal by definition;
 * keys >= q0 + nq. Key tiles wholly below the window are neither loaded nor multiplied; the decode splits
 * share only the window's keys. Workspace as for mb_attention (its size is an upper bound here). */
int mb_attention_window(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v, size_t batch,
                        size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                        size_t window, void* out, void* workspace, size_t workspace_bytes);

/* Causal decode attention with the remaining terms of flash_attention_kernel
 * (src/models/inkling/flash.rs:751-785): a relative bias and eviction gaps.
 * rel (or NULL): [batch, nq, heads, eff] f32; a visible key at distance dist = q_abs - k_abs < eff
 * gets rel[.., dist] added to its scaled score. gap_rows / gap_cums (ngaps <= 64 device words each,
 * rows ascending; or NULL, 0): the key in cache row r sits at position r + gap_cums[g] for the last g
 * with gap_rows[g] <= r, at r when there is none; visibility, the window and the bias distance all
 * use positions, and q0 is the position of the first query. All sequences of a call share the gap
 * list. window = 0: none. Decode shapes (nq * heads / kv_heads <= 16) run on the split-K decode kernel;
 * prompt-shaped blocks run on the warp-level (mma.sync) prompt kernel, which masks and biases every score
 * by position (correct at any nq, at about a fifth of the tcgen05 kernel's rate). */
int mb_attention_decode_ext(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v, size_t batch,
                            size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                            size_t window, const float* rel, size_t eff, const uint32_t* gap_rows,
                            const uint32_t* gap_cums, size_t ngaps, void* out, void* workspace, size_t workspace_bytes);

/* Decode attention over an NVFP4 key/value cache: the packed reader of flash_attention_kernel
 * (`nvfp4_at`, src/models/inkling/flash.rs:520-540, 827-859) over the Fp4Rows page layout
 * (src/models/inkling/kvpages.rs:1378-1404): a cache row of kv_heads * D features is quantized
 * row-major in blocks of 16 along the features with no global scale, i.e. the bytes
 * mb_nvfp4_quantize_act(MB_QUANT_RECIP, row-major scales) writes for the [keys, kv_heads * D]
 * rows. codes [batch, keys, kv_heads * D / 2], scales [batch, keys, kv_heads * D / 16].
 * A value is E2M1[code] * e4m3(scale), exact in f16: the kernel expands rows to f16 and runs
 * both products as f16 x f16 with f32 accumulation (Q converted to f16, probabilities kept
 * to 11 bits), reading 0.5625 bytes per cached value instead of 2. The result agrees with
 * mb_attention (mb_attention_window when window > 0) over the dequantized rows to a bf16 step
 * of the output. Decode shapes only
 * (nq * heads / kv_heads <= 16); workspace as for mb_attention. Codes 16-byte, scales 8-byte aligned. */
int mb_attention_fp4kv(mb_ctx* ctx, mb_stream stream, const void* q, const uint8_t* k_codes, const uint8_t* k_scales,
                       const uint8_t* v_codes, const uint8_t* v_scales, size_t batch, size_t nq, size_t keys,
                       size_t heads, size_t kv_heads, size_t d, size_t q0, float scale, int causal, size_t window,
                       void* out, void* workspace, size_t workspace_bytes);

/* flash_attention_launch (src/models/inkling/flash.rs:1140-1316) with its own argument list: one query
 * block over any number of key runs, one run per page of a paged cache (KeyRun, flash.rs:995-1015).
 * A run's buffers hold `rows` rows per sequence ([batch, rows, kv_heads * D], token-major; batch = 1 is
 * the reference's call, more are independent sequences with identical run geometry); `base` is the
 * absolute position of row 0; rows [lo, hi) are live keys (a page's dropped prefix and its tail padding
 * are excluded without slicing the buffer); `row0` is the logical row of stored row 0, which the gap
 * table is indexed by. kv_elem (KvElem, flash.rs:972-981): MB_KV_BF16 rows are read in place by TMA;
 * MB_KV_NVFP4 runs carry code bytes in k/v ([.., kv_heads * D / 2]) and E4M3 block scales in
 * k_scales/v_scales ([.., kv_heads * D / 16]) and are read packed; MB_KV_F32 rows are rounded to bf16
 * into the workspace first (both products multiply bf16). q [batch, nq, heads * D] and out likewise,
 * each bf16 or f32 (the reference's are f32); query i stands at absolute position q0 + i. Always causal
 * on positions: a key is visible when key_abs <= q_abs, within `window` when window > 0
 * (q_abs - key_abs < window), and gets rel[.., dist] added at distance dist < eff (rel [batch, nq, heads,
 * eff] f32 or NULL). gap_rows/gap_cums (ngaps <= 64 device words each, or NULL, 0): the eviction gaps of
 * Gaps (flash.rs:1017-1035). Decode shapes (nq * heads / kv_heads <= 16) split every run's visible keys
 * in proportion to its span (key_run_splits, flash.rs:1318-1327) and merge all partials in one pass;
 * prompt shapes take a single non-empty run and run on the tcgen05 kernel (on the warp-level kernel when they
 * carry a bias or gaps); NVFP4
 * rows reach it through the dequantizing reader (flash.rs:520-540): the run's live rows are expanded to
 * bf16 in the workspace, exactly. At most 64 runs. workspace: mb_attention_runs_workspace bytes, 256-byte
 * aligned. */
enum { MB_KV_F32 = 0, MB_KV_BF16 = 1, MB_KV_NVFP4 = 2 };
typedef struct mb_key_run {
  const void* k;
  const void* v;
  const void* k_scales; /* MB_KV_NVFP4 only, else NULL */
  const void* v_scales;
  size_t rows;          /* rows per sequence in the buffers */
  size_t base;          /* absolute sequence position of row 0 */
  size_t lo;            /* first live row */
  size_t hi;            /* one past the last live row */
  size_t row0;          /* logical row of stored row 0 (gap table index) */
} mb_key_run;
size_t mb_attention_runs_workspace(const mb_key_run* runs, size_t n_runs, int kv_elem, size_t batch, size_t nq,
                                   size_t q0, size_t heads, size_t kv_heads, size_t d, size_t window, size_t ngaps,
                                   int q_dtype, int out_dtype);
int mb_attention_runs(mb_ctx* ctx, mb_stream stream, const void* q, int q_dtype, const mb_key_run* runs, size_t n_runs,
                      int kv_elem, const float* rel, size_t eff, const uint32_t* gap_rows, const uint32_t* gap_cums,
                      size_t ngaps, size_t batch, size_t nq, size_t q0, size_t heads, size_t kv_heads, size_t d,
                      size_t window, float scale, void* out, int out_dtype, void* workspace, size_t workspace_bytes);

/* Decode attention without any allocation; it has no counterpart in the reference.
 * For hosts that gave all device memory to their own arena at start-up and may not
 * call the driver's allocator afterwards (an allocation there stalls the token step
 * and can fail under a full arena): the key-split scratch lives in a 16 MiB array
 * built into the library, so the caller passes only q, k, v and out. Same arithmetic
 * and argument meaning as mb_attention for decode shapes (nq * heads/kv_heads <= 16);
 * it splits the keys less than mb_attention would when that is what fits the array.
 * The array is also the entry point's one stated limit: a shape whose partials would not
 * fit it at a single split (batch * kv_heads > 2016) is refused with MB_ERR_INVALID, by
 * policy, although an unsplit launch would not use the array.
 * The array and the two kernels become resident in mb_ctx_create (which runs
 * mb_attention_decode_static_warm: address look-up, function attributes and one tiny
 * launch of each kernel inside the array), not at the first call: create the contexts
 * before the host sizes its arena, and before any stream capture. All calls share the one
 * array: the partials are fully rewritten by every call, nothing needs clearing, but two
 * calls that overlap on the GPU (different streams) race on it. */
int mb_attention_decode_static_warm(mb_ctx* ctx);
int mb_attention_decode_static(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v,
                               size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d,
                               size_t q0, float scale, int causal, void* out);

/* ---- decoder-layer glue (Breeze rounding points) ------------------------------------ */
/* norm_kernel (src/models/breeze/cuda_ops.rs:88-117): bf16(bf16(x*inv)*gain). */
int mb_rmsnorm(mb_ctx* ctx, mb_stream stream, const void* x_bf16, const void* gain_bf16, size_t rows,
               size_t width, float eps, void* out_bf16);
/* rms_norm_kernel (src/models/inkling/resid.rs:272-322), the Inkling convention: f32 throughout and ONE
 * rounding, out = O(x / sqrt(mean(x^2) + eps) * gain) with an f32 gain [width]; x and out bf16 or f32.
 * The sum of squares runs in the reference kernel's order (min(256, next power of two of width) strided
 * partials, then a halving tree), so the result does not depend on scheduling. width % 8 == 0, <= 8192. */
int mb_rmsnorm_inkling(mb_ctx* ctx, mb_stream stream, const void* x, int x_dtype, const float* gain_f32, size_t rows,
                       size_t width, float eps, void* out, int out_dtype);
/* gate_up_silu(_narrow/_bf16)_launch (src/models/inkling/fp4gemm.rs:472-507, 574-623): the stand-alone pass
 * over a fused gate/up result both [rows, 2 * inter] (bf16 or f32): act[r, i] = O(silu(g) * u) computed in
 * f32, (g, u) = columns (2i, 2i + 1) when the rows of w13 interleave, columns (i, inter + i) when
 * `halved` (all gates, then all ups). inter % 4 == 0. */
int mb_gate_up_silu(mb_ctx* ctx, mb_stream stream, const void* both, int in_dtype, size_t rows, size_t inter,
                    int halved, void* act, int out_dtype);
/* element_kernel mode 0 / mode 2 (src/models/breeze/cuda_ops.rs:230-255). */
int mb_add(mb_ctx* ctx, mb_stream stream, const void* a_bf16, const void* b_bf16, size_t n, void* out_bf16);
int mb_swiglu(mb_ctx* ctx, mb_stream stream, const void* gate_bf16, const void* up_bf16, size_t n,
              void* out_bf16);
/* The residual add after a tensor-parallel reduction: out = bf16(a + bf16(partial_sum_f32)).
 * The all-reduced partial is f32 (src/models/inkling/tpcomm.rs:1453-1467); rounding it to bf16
 * first reproduces add(x, linear(..)) of src/models/breeze/backbone.rs:326-329 at world 1. */
int mb_add_f32(mb_ctx* ctx, mb_stream stream, const void* a_bf16, const float* b_f32, size_t n, void* out_bf16);
/* rope_kernel (src/models/breeze/cuda_ops.rs:286-320): x [tokens, heads, d], in place allowed. */
int mb_rope(mb_ctx* ctx, mb_stream stream, const void* x_bf16, size_t tokens, size_t heads, size_t d,
            size_t past, const float* inv_freq, void* out_bf16);

/* The same glue with fewer passes over the activations; every value is computed by the
 * arithmetic, in the order, of the separate entry points above, so the bytes are the same.
 *
 * mb_residual_norm_quantize: [r = bf16(resid + bf16(partial)), stored to resid_out, when a
 * partial f32 sum is given, else r = resid;] y = rmsnorm(r, gain) as mb_rmsnorm; y goes out as
 * W4A4 activation planes (codes [rows, width/2], tiled scale plane) as mb_nvfp4_quantize_act
 * with MB_QUANT_SCALED and input_scale 1 writes them. width % 64 == 0, width <= 8192.
 * The chain add_bf16 -> RmsNorm::forward -> quantize of src/nn/nvfp4_gemm.rs:644-669. */
int mb_residual_norm_quantize(mb_ctx* ctx, mb_stream stream, const void* resid, const float* partial, const void* gain,
                              size_t rows, size_t width, float eps, void* resid_out, uint8_t* codes,
                              uint8_t* sf_tiled);

/* mb_rope_append: qkv is a stacked projection [batch * t, (hq + 2 hkv) * d] bf16 (sequence
 * major, t new tokens per sequence at positions past .. past + t). q heads are rotated into
 * q_out [batch * t, hq * d]; k heads are rotated and v heads copied into the caches
 * [batch, capacity, hkv, d] at [past, past + t). Per element it is mb_rope. d % 16 == 0. */
int mb_rope_append(mb_ctx* ctx, mb_stream stream, const void* qkv, size_t batch, size_t t, size_t hq, size_t hkv,
                   size_t d, size_t past, const float* inv_freq, void* q_out, void* k_cache, void* v_cache,
                   size_t capacity);

/* ---- tensor parallel ---------------------------------------------------------------- */
/* Tp::shard (src/models/inkling/tp.rs:540-555). Host arithmetic only. */
int mb_tp_shard(size_t rank, size_t world, size_t extent, size_t* lo, size_t* hi);
/* Group::form / warm / all_reduce_f32 (src/models/inkling/tpcomm.rs:271-310,
 * 377-404, 415-429): rank 0 mints a 128-byte NCCL id, every rank joins with it;
 * warm() all-reduces ones and requires the sum to equal world. */
int mb_tp_unique_id(mb_ctx* ctx, uint8_t id_out[128]);
int mb_tp_form(mb_ctx* ctx, const uint8_t id[128], int rank, int world);
int mb_tp_warm(mb_ctx* ctx, mb_stream stream);
int mb_tp_all_reduce(mb_ctx* ctx, mb_stream stream, void* buf, size_t count, int dtype);
/* The two halves of that all-reduce for prompt-sized activations (no counterpart in the reference, which
 * all-reduces the whole f32 partial, src/models/inkling/tpcomm.rs:1453-1467): SUM reduce-scatter of the f32
 * partial by rows, so each rank adds the residual, normalises and quantizes only its own rows, then an
 * all-gather of what the next product reads (NVFP4 planes: 0.5625 bytes per element instead of 4). The sums
 * are the all-reduce's f32 sums; only who holds which rows in between differs. send holds world x recv_count
 * floats; mb_tp_all_gather moves raw bytes and works in place when send == recv + rank * send_bytes. */
int mb_tp_reduce_scatter_f32(mb_ctx* ctx, mb_stream stream, const float* send, float* recv, size_t recv_count);
int mb_tp_all_gather(mb_ctx* ctx, mb_stream stream, const void* send, void* recv, size_t send_bytes);
int mb_tp_close(mb_ctx* ctx);

/* Fused row-parallel path over peer memory: tp_reduce (src/models/inkling/tpcomm.rs:1453-1467)
 * + the residual add that follows it (src/models/inkling/session.rs:2713-2717, 2793, 2843-2846,
 * 2930), as one exchange that overlaps the GEMM. Each rank creates exchange memory for activations
 * up to [t_max, n] (mb_tp_symm_create returns a 64-byte CUDA IPC handle), the handles of all ranks
 * travel over the host link in rank order, and mb_tp_symm_attach maps them. Per reduction, with a
 * step counter that grows by one each time (from 1): mb_nvfp4_gemm_w4a4_scatter is
 * mb_nvfp4_gemm_w4a4 whose epilogue pushes each f32 partial tile into the rank owning those
 * columns (reduce-scatter by peer stores); mb_tp_reduce_residual then sums this rank's columns
 * in rank order, forms bf16(resid + bf16(sum)), stores it into every rank's output (all-gather by
 * peer stores) and returns the device address of the local [t, n] bf16 result, valid until the
 * step after next. Waits on peers are bounded (status word on timeout). world <= 8. */
size_t mb_tp_symm_bytes(size_t t_max, size_t n);
int mb_tp_symm_create(mb_ctx* ctx, size_t t_max, size_t n, uint8_t handle_out[64]);
int mb_tp_symm_attach(mb_ctx* ctx, const uint8_t* handles_world_x64, int rank, int world);
/* The same for ranks that live in ONE process (the reference's Group is threads of one process,
 * src/models/inkling/tpcomm.rs:217-310): mb_tp_symm_local gives the device address of this context's
 * exchange memory, and mb_tp_symm_attach_ptrs takes every rank's address as this process sees it
 * (peers[rank] is ignored; peer access between the devices is the caller's to enable). */
int mb_tp_symm_local(mb_ctx* ctx, void** local_out);
int mb_tp_symm_attach_ptrs(mb_ctx* ctx, void* const* peers, int rank, int world);
int mb_nvfp4_gemm_w4a4_scatter(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                               const uint8_t* b_codes, const uint8_t* b_sf_tiled, float alpha, size_t m, size_t n,
                               size_t k, int step);
int mb_tp_reduce_residual(mb_ctx* ctx, mb_stream stream, const void* resid_bf16, size_t t, size_t n, int step,
                          void** out_dev);
int mb_tp_symm_destroy(mb_ctx* ctx);

/* The same two halves (reduce-scatter by rows, all-gather) as kernels of this library over peer memory, for
 * prompt-sized messages: tp_reduce's sums (src/models/inkling/tpcomm.rs:1453-1467) with this rank's rows left
 * local in between. Each rank creates a region of mb_tp_bulk_header_bytes() + user_bytes (64-byte CUDA IPC
 * handle out), the handles travel over the host link in rank order, mb_tp_bulk_attach maps them
 * (mb_tp_bulk_attach_ptrs for ranks of one process); mb_tp_bulk_local gives the region's address and that of
 * its user part, in which the caller lays out receive areas and gathered buffers by byte offset (256-byte
 * aligned), the same on every rank.
 * mb_tp_bulk_reduce_scatter_f32: every rank's partial [rows, n] f32 lies at partial_off in its own region (its
 * row-parallel product wrote it there), rows % world == 0; a rank reads its own rows out of every rank's partial
 * with peer loads and this rank's rows of the sum, added in rank order, land in out [rows / world, n] (local).
 * mb_tp_bulk_all_gather: for up to two buffers at off0 / off1 whose rank-th slice of
 * part_bytes the caller has already written in its OWN region, the slice is pushed to the same place on every
 * peer and the call's kernel ends when all slices have arrived (part_bytes1 = 0: one buffer).
 * `step` counts the calls of each kind from 1, the same on every rank, and the calls of a kind run in that order
 * (issue them on one stream). A partial or a gathered buffer may be written again two calls of its kind later
 * (alternate between two). Waits on peers are bounded by the context's
 * wait limit; a wait that runs out leaves status 54 / 55 (mb_check_flags) and the context usable. world <= 8. */
size_t mb_tp_bulk_header_bytes(void);
int mb_tp_bulk_create(mb_ctx* ctx, size_t user_bytes, uint8_t handle_out[64]);
int mb_tp_bulk_attach(mb_ctx* ctx, const uint8_t* handles_world_x64, int rank, int world);
int mb_tp_bulk_attach_ptrs(mb_ctx* ctx, void* const* peers, int rank, int world);
int mb_tp_bulk_local(mb_ctx* ctx, void** region_out, void** user_out);
int mb_tp_bulk_reduce_scatter_f32(mb_ctx* ctx, mb_stream stream, size_t partial_off, size_t rows, size_t n, float* out,
                                  int step);
int mb_tp_bulk_all_gather(mb_ctx* ctx, mb_stream stream, size_t off0, size_t part_bytes0, size_t off1,
                          size_t part_bytes1, int step);
int mb_tp_bulk_destroy(mb_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* MARY_B200_H */
