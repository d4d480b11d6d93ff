/*
 * lkb.h - C ABI of the B200 (sm_100a) Q4_0 x Q8_1 MoE hot path.
 *
 * One entry point per kernel (or host launcher) of the reference engine's hot
 * path.  Each takes the reference kernel's own parameter list -- same order,
 * same meaning -- followed by the CUDA stream to launch on, and returns an int
 * status (LKB_OK, or a negative LKB_ERR_* / -cudaError_t) instead of exiting the
 * process.  Grid and block shapes are chosen inside.  All pointers are DEVICE
 * pointers owned by the caller; nothing here allocates device memory, blocks the
 * host or synchronises the stream, so every call may be captured into a CUDA
 * graph (after lkb_init() has run once for the device).
 *
 * "ref:" comments give the reference interface an entry point replaces, as
 * <file>:<line> relative to the reference repository (Nathan-T-Ray/lfm2-ampere).
 *
 * Data formats (identical to the reference's planar pack):
 *   Q4_0 weights   qs plane: 16 bytes per 32-element block, byte j = element j
 *                  (low nibble) | element j+16 (high nibble), nibbles unsigned;
 *                  d plane: one fp16 scale per block.  Row-major [row][bpr];
 *                  the experts of one tensor are stacked: row = e*rows_per_expert + r.
 *                  ref: src/quant.cuh:4-9,124-130
 *   block_q8_1     36 bytes: {fp16 d = amax/127, fp16 s = raw sum, int8 qs[32]}.
 *                  ref: src/quant.cuh:27-31
 *   planar Q8_1    lkb_pf_act: qs int8 [rows][kb*32], sc float2 [rows][kb] with
 *                  .x = float(fp16 d), .y = 8*float(fp16 sum).  ref: src/prefill.cuh:27-36
 */
#ifndef LKB_H
#define LKB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)   /* the entry points below are the library's whole export list */
#endif

#define LKB_OK               0
#define LKB_ERR_SHAPE       -10001   /* a documented shape precondition is violated */
#define LKB_ERR_NULL        -10002   /* a required pointer is null */
#define LKB_ERR_UNSUPPORTED -10003   /* a mode of the reference that this build leaves out */
#define LKB_ERR_NOT_INIT    -10004   /* lkb_init() has not run for the current device */
#define LKB_ERR_DEVICE      -10005   /* not an sm_100 device */
#define LKB_ERR_TIMEOUT     -10006   /* a bounded device-side wait gave up (status word set) */
#define LKB_ERR_SCRATCH     -10007   /* the shape needs more scratch than the library's built-in array holds */

/* Model constants of the path.  ref: src/kernels.cuh:11-24 */
#define LKB_HIDDEN      2048
#define LKB_N_EXPERTS   64
#define LKB_TOP_K       4
#define LKB_MOE_INTER   1536
#define LKB_EPS         1e-5f
#define LKB_TOPK_GUARD  6.103515625e-5f
#define LKB_MOE_BN      64           /* token tile of the MoE plan.  ref: src/prefill.cuh:72 */

typedef struct CUstream_st * lkb_stream_t;          /* == cudaStream_t */

typedef struct { uint16_t d, s; int8_t qs[32]; } lkb_block_q8_1;   /* 36 bytes */

/* ref: src/kernels.cuh:413-418 (LKNormProd) */
typedef struct {
    const float *    w;      /* norm weights to apply, or null: no producer step */
    float *          h32;    /* raw x*w in fp32 (router input), or null */
    lkb_block_q8_1 * yq8;    /* quantised RAW activation x*w */
    float *          ssq;    /* [64] per-block sums of squares of x */
} lkb_norm_prod_t;

/* ref: src/prefill.cuh:33-36 (PfAct) */
typedef struct {
    int8_t * qs;
    float *  sc;             /* float2 per block */
} lkb_pf_act;

/* ref: src/prefill.cuh:45-66 (PfGemm); tiles entries are int4 {expert, start, count, 0} */
typedef struct {
    const void *   qs[3];        /* uint4 per block */
    const void *   d[3];         /* fp16 per block */
    int            seg_end[3];   /* cumulative row ends, multiples of 128 */
    int            N;            /* output rows (features): multiple of 128 (64 for the SwiGLU form) */
    int            bpr;          /* 32-element blocks per row, multiple of 8 */
    long long      exp_stride;   /* blocks per expert, 0 if dense */
    const int8_t * aqs;          /* activations, row pitch bpr*32 */
    const float *  asc;          /* float2 [rows][bpr] */
    int            ntok;         /* dense: token rows */
    const int *    perm;         /* MoE: slot ids grouped by expert, or null */
    const int *    tiles;        /* MoE: int4 {expert, start in perm, count, 0} */
    const int *    ntiles;       /* MoE: device-side tile count */
    int            a_shift;      /* activation row = slot >> a_shift */
    const float *  scale;        /* per activation row, or null */
    float *        out;
    int            out_ld;
    int            add;          /* 1: out += result */
    int8_t *       oqs;          /* SwiGLU form only: planar Q8_1 output */
    float *        osc;
    int            okb;
} lkb_pf_gemm;

/* ------------------------------------------------------------------ set-up */
/* One-time per device: checks for sm_100, records the SM count, sets the
 * dynamic shared-memory limits of the kernels.  Not part of the reference
 * (its launchers do this lazily behind function-local statics,
 * ref: src/prefill.cu:705-709); call it before any stream capture. */
int lkb_init(int device);
const char * lkb_error_string(int status);
int lkb_sm_count(void);
/* 1: launch the decode kernels with programmatic dependent launch so that a
 * kernel's weight prefetch overlaps its predecessor's tail.  Default 0. */
int lkb_set_pdl(int enable);

/* ------------------------------------------------- activation quantisers */
/* ref: src/kernels.cuh:73-74  k_quantize_q8_1<<<nblocks,32>>> */
int lkb_quantize_q8_1(const float * x, lkb_block_q8_1 * y, int nblocks, lkb_stream_t st);
/* ref: src/kernels.cuh:66-68  k_rmsnorm_q8_1<<<1,256>>>; n must be 2048; y16 is fp16 */
int lkb_rmsnorm_q8_1(const float * x, const float * w, int n, float eps, float * y32,
                     void * y16, lkb_block_q8_1 * yq8, lkb_stream_t st);
/* The stand-alone producer of the scale-carrying norm split: quantise x*w, emit
 * ssq[64] (and h32).  ref: src/kernels.cuh:421-431 (lk_norm_prod_warp, called by
 * k_moe_accum4 with a zero contribution); n must be a multiple of 32. */
int lkb_norm_produce(const float * x, int n, const lkb_norm_prod_t * np, lkb_stream_t st);

/* ------------------------------------------------------------ decode GEMVs */
/* ref: src/kernels.cuh:449-452  k_gemv_q4_0 */
int lkb_gemv_q4_0(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                  float * y, int add_residual, const float * ssq, float eps, lkb_stream_t st);
/* ref: src/kernels.cuh:457-460  k_gemv_q4_0_prod; out_rows % 32 == 0 */
int lkb_gemv_q4_0_prod(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                       float * y, int add_residual, const lkb_norm_prod_t * np, lkb_stream_t st);
/* ref: src/kernels.cuh:704-711  k_gemv_q4_0_3 */
int lkb_gemv_q4_0_3(const void * qs0, const void * d0, int rows0, float * y0,
                    const void * qs1, const void * d1, int rows1, float * y1,
                    const void * qs2, const void * d2, int rows2, float * y2,
                    const lkb_block_q8_1 * xq, int bpr, const float * ssq, float eps, lkb_stream_t st);
/* ref: src/kernels.cuh:713-722  k_gemv_q4_0_exp2.  The router-in-prologue group
 * (sel, sig, idx_out, w_out; off by default in the reference) must be null. */
int lkb_gemv_q4_0_exp2(const void * qs_a, const void * d_a, const void * qs_b, const void * d_b,
                       const lkb_block_q8_1 * xq, int out_rows, int bpr, int rows_per_expert, int xq_stride,
                       const int * d_idx, const float * sel, const float * sig, int * idx_out, float * w_out,
                       float * y_a, float * y_b, const float * ssq, float eps, lkb_stream_t st);
/* ref: src/kernels.cuh:724-731  k_gemv_q4_0_exp */
int lkb_gemv_q4_0_exp(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                      int rows_per_expert, int xq_stride, const int * d_idx, float * y, lkb_stream_t st);
/* ref: src/kernels.cuh:476-481  k_swiglu (n % 32 == 0).  pf_* describe the
 * down-projection weights to pull towards L2 while the activation is built. */
int lkb_swiglu(const float * gate, const float * up, int n, float * out, lkb_block_q8_1 * yq8,
               const void * pf_qs, const int * pf_idx, int pf_rows_per_expert, int pf_bpr, long pf_bytes,
               lkb_stream_t st);
/* ref: src/kernels.cuh:733-734  k_moe_accum4 */
int lkb_moe_accum4(float * dst, const float * down4, const float * d_w, int n, const lkb_norm_prod_t * np,
                   lkb_stream_t st);
/* ref: src/kernels.cuh:735-739  k_moe_down_accum; out_rows % 32 == 0 */
int lkb_moe_down_accum(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                       int rows_per_expert, int xq_stride, const int * d_idx, const float * d_w,
                       float * dst, const lkb_norm_prod_t * np, lkb_stream_t st);

/* ------------------------------------------------ fused MoE FFN (decode) */
/* One MoE layer's tensors (device pointers into the planar pack). */
typedef struct {
    const void *  gate_qs; const void * gate_d;     /* [64*1536][64] blocks */
    const void *  up_qs;   const void * up_d;
    const void *  down_qs; const void * down_d;     /* [64*2048][48] blocks */
    const float * router;                           /* [64][2048] */
    const float * rbias;                            /* [64] or null */
    const float * norm_w;                           /* [2048] ffn_norm weights */
    int           softmax;                          /* 0: sigmoid+bias gate (the reference's); 1: softmax gate */
} lkb_moe_layer;
/* The fused kernels read x, the norm weights (ffn_norm, attn_norm, the optional final norm) and the scratch vectors 128
 * bits at a time: those pointers must be 16-byte aligned (LKB_ERR_SHAPE where the launcher can see them).
 * Caller-owned global scratch of the fused kernels: 64 floats (router logits), 2*4*1536 floats (exchange of the
 * intermediate activations; the current kernels use the first 4*1536) and
 * two 32-bit words (barrier counter, status; status != 0 after the kernel means a
 * bounded wait expired: 1000+10*layer+n = grid barrier n, 100/200/300+layer = a copy). */
#define LKB_MOE_SCRATCH_LOGITS 64
#define LKB_MOE_SCRATCH_GU     (2 * LKB_TOP_K * LKB_MOE_INTER)
#define LKB_MOE_SCRATCH_SYNC   2
typedef struct {
    float *    logits;
    float *    gu;
    unsigned * sync;
} lkb_moe_scratch;
/* Sequence mixer of one layer for the whole-step kernel (lkb_decode_layers): the short convolution
 * (is_attn == 0: in_proj 6144 x 2048, conv taps, two-tap history, out_proj) or GQA attention (is_attn != 0:
 * q / k / v projections 2048 / 512 / 512 x 2048, per-head norm weights, this layer's fp16 KV cache,
 * attn_output).  All weight planes are Q4_0 planar (qs, d) with 64 blocks per row.
 * ref: src/engine.cu:136-145 (struct Layer) */
typedef struct {
    int           is_attn;
    int           max_seq;                          /* attention: positions the KV cache holds; 0 = not checked.  A step at
                                                     * *d_pos >= max_seq writes nothing and sets status 600 + layer */
    const float * attn_norm;                        /* fp32[2048], the norm in front of the mixer */
    const void *  in_qs;  const void * in_d;        /* conv: in_proj */
    const float * conv_w;                           /* conv: fp32[2048*3] */
    float *       hist;                             /* conv: fp32[2048*2], updated in place */
    const void *  wq_qs;  const void * wq_d;
    const void *  wk_qs;  const void * wk_d;
    const void *  wv_qs;  const void * wv_d;
    const float * qnorm;  const float * knorm;      /* fp32[64] each */
    void *        kc;     void * vc;                /* fp16 [max_seq][8][64] */
    const void *  out_qs; const void * out_d;       /* out_proj / attn_output, 2048 x 2048 */
} lkb_mixer_layer;
/* Caller-owned global scratch of the whole-step kernel, beside lkb_moe_scratch. */
#define LKB_STEP_SCRATCH_MX   3072                  /* floats: q | k | v of an attention layer, or the conv output */
#define LKB_STEP_SCRATCH_PART (32 * 18 * 66)        /* floats: attention partials */
typedef struct {
    float * mx;
    float * part;
} lkb_step_scratch;
/* One launch for one batch-1 MoE FFN layer: x (the residual stream, fp32[2048]) is
 * normalised-and-quantised with layer->norm_w, routed, pushed through the four chosen
 * experts and updated in place; idx_out/w_out (optional) receive the selection; `next`
 * (optional, w != null) receives the quantised raw activation, ssq and h32 of the new x
 * for the caller's next consumer.  Bit-identical to the sequence lkb_norm_produce ->
 * lkb_router_dot -> lkb_router_top4 -> lkb_gemv_q4_0_exp2 -> lkb_swiglu ->
 * lkb_moe_down_accum.  No counterpart in the reference: it fuses the five launches of
 * ref: src/engine.cu:739-811 into a persistent cooperative kernel (one CTA per SM). */
int lkb_moe_ffn_decode(const lkb_moe_layer * layer, float * x, int * idx_out, float * w_out,
                       const lkb_norm_prod_t * next, const lkb_moe_scratch * scratch, lkb_stream_t st);
/* Expert prefetch of the multi-layer kernels (bit 0: lkb_moe_ffn_decode_stack[_static], bit 1: lkb_decode_layers;
 * sigmoid gate, at least 128 CTAs).  While layer l runs, 64 CTAs that have no router row of their own evaluate layer
 * l+1's router on layer l's input, and each CTA, once its rows of layer l have arrived, asks for its slice of the four
 * guessed experts of layer l+1 to be brought into L2 (cp.async.bulk.prefetch.L2).  Results are unchanged bit for bit:
 * the exact selection decides what is computed, a wrong guess only costs idle HBM bandwidth.  The guesses and the actual
 * choices of the last launch are kept in the second half of scratch->gu; lkb_decode_expert_prefetch_hits waits for
 * `st` and counts how many of the 4*(n_layers-1) guesses were chosen.  The idea of warming L2 with expert rows ahead of
 * their use is the reference's (ref: src/kernels.cu:499-510, there for the current layer's down rows).
 * Off by default (mode 0): on B200, with 74-81% of the guesses chosen, a 40-layer step measured 2-4% slower with it. */
int lkb_decode_set_expert_prefetch(int mode);
int lkb_decode_expert_prefetch_hits(const lkb_moe_scratch * scratch, int n_layers, int * hits, int * guesses, lkb_stream_t st);
/* The same for n_layers consecutive layers in ONE launch; layers_dev is a DEVICE array
 * of descriptors; idx_out/w_out (optional) are [n_layers][4].  No counterpart in the
 * reference (its decode step is a 343-node graph, ref: src/engine.cu:1336-1342). */
int lkb_moe_ffn_decode_stack(const lkb_moe_layer * layers_dev, int n_layers, int softmax, float * x,
                             int * idx_out, float * w_out, const lkb_norm_prod_t * next,
                             const lkb_moe_scratch * scratch, lkb_stream_t st);

/* All n_layers layers of a batch-1 decode step in ONE persistent launch: per layer the sequence mixer
 * (mixers_dev[l]) and the MoE FFN (moe_dev[l]), with x the residual stream updated in place.  xq_first is
 * layer 0's normalised Q8_1 activation (from lkb_rmsnorm_q8_1 with layer 0's attn_norm); every later norm is
 * evaluated inside.  Attention layers read the position from *d_pos, append the new K / V row to their cache
 * and attend over positions 0..*d_pos.  `next` (w != null) receives the quantised raw activation and ssq of
 * the final x for the output projection.  Results are bit-identical to the kernel-by-kernel sequence
 * (lkb_gemv_q4_0 / lkb_shortconv / lkb_gemv_q4_0_3 / lkb_qk_norm_rope / lkb_attn_split / lkb_attn_combine /
 * lkb_gemv_q4_0_prod, then the MoE kernels).  Status word as for lkb_moe_ffn_decode (400/500+layer = a mixer
 * copy, 1000+10*layer+n = grid barrier n).  No counterpart in the reference (its step is a 343-node graph,
 * ref: src/engine.cu:1336-1342). */
int lkb_decode_layers(const lkb_moe_layer * moe_dev, const lkb_mixer_layer * mixers_dev, int n_layers, float * x,
                      const lkb_block_q8_1 * xq_first, const int * d_pos, float theta, const lkb_norm_prod_t * next,
                      const lkb_moe_scratch * scratch, const lkb_step_scratch * step_scratch, lkb_stream_t st);

/* lkb_moe_ffn_decode_stack for callers that must not allocate device memory.
 * Who that is: an engine that, like the reference's, sizes one pack allocation plus its KV cache at start-up
 * and hands the rest of the card to someone else; a plug-in living inside a host process whose memory pool
 * owns every byte (a foreign cudaMalloc there fragments the pool or is simply forbidden); a latency-critical
 * decode loop, where cudaMalloc/cudaFree would stall the whole device at an unpredictable moment.  Such a
 * caller still owns its inputs and outputs (layers_dev, x, idx_out, w_out, next) but has nowhere to put the
 * kernel's scratch, so here the scratch -- 64 router logits, the 2*4*1536 gate|up outputs and two barrier
 * words, 49.7 KB for this model -- sits in a fixed LKB_STATIC_SCRATCH_BYTES array inside the library (every
 * GPU that loads the library carries that array until the process exits).
 * The caller states its model shape; a shape whose scratch does not fit the array is refused with
 * LKB_ERR_SCRATCH, and a shape other than the one the kernel is built for (2048 / 1536 / 64 / 4) with
 * LKB_ERR_SHAPE.  Nothing is allocated or freed, by this call or by anything it calls.
 * The first call on a device looks up the array's device address (once per device, with that device
 * current); make that first call outside any stream capture.  All calls share the one array, which keeps
 * whatever the previous call left in it: the barrier words are cleared at the start of every call, the rest
 * is overwritten before it is read.  Two calls that overlap on the GPU (different streams) race on it.
 * No counterpart in the reference. */
#define LKB_STATIC_SCRATCH_BYTES 65536
#define LKB_STATIC_MAX_DEVICES   64
int lkb_moe_ffn_decode_stack_static(const lkb_moe_layer * layers_dev, int n_layers, int hidden, int inter,
                                    int n_experts, int top_k, int softmax, float * x, int * idx_out, float * w_out,
                                    const lkb_norm_prod_t * next, lkb_stream_t st);
/* The bounded-wait status of the last lkb_moe_ffn_decode_stack_static call on the current device: 0, or the code of
 * the device-side wait that gave up (what a caller of the allocating form reads from scratch->sync[1] itself; here
 * the word lives in the library's array).  SYNCHRONISES the device, copies four bytes, allocates nothing.
 * No counterpart in the reference. */
int lkb_moe_ffn_decode_stack_static_status(void);

/* ------------------------------------------------------------------ router */
/* ref: src/kernels.cuh:543-547  k_router_dot<<<64,32>>> (sel/sig may be null) */
int lkb_router_dot(const float * h, const float * gate_inp, float * logits, const float * bias,
                   float * sel, float * sig, const float * ssq, float eps, lkb_stream_t st);
/* ref: src/kernels.cuh:548-550  k_router_top4<<<1,64>>> */
int lkb_router_top4(const float * logits, const float * bias, int * idx_out, float * w_out, lkb_stream_t st);
/* Softmax gate of the synthetic configurations: p = softmax(logits), ranking by
 * p + bias (bias may be null), weights p renormalised over the top four.  No
 * counterpart in the reference (its gate is the sigmoid above). */
int lkb_router_top4_softmax(const float * logits, const float * bias, int * idx_out, float * w_out,
                            lkb_stream_t st);

/* ------------------------------------------------------------ debug taps */
/* Integer block sums S[row][blk] = sum_i nibble_i * q_i of one activation row
 * against a [rows][bpr] matrix.  No counterpart in the reference; it exposes the
 * int32 value inside dot_q4_0_q8_1 (ref: src/quant.cuh:141-151) for parity tests. */
int lkb_block_sumi(const void * qs, const lkb_block_q8_1 * xq, int rows, int bpr, int32_t * out,
                   lkb_stream_t st);

/* ----------------------------------------------------------------- prefill */
/* ref: src/prefill.cuh:81-82  k_pf_norm<<<m,256>>> */
int lkb_pf_norm(const float * X, const float * w, int plain, lkb_pf_act a, float * inv_out, float * h32,
                int m, lkb_stream_t st);
/* ref: src/prefill.cuh:107  k_pf_quant_rows */
int lkb_pf_quant_rows(const float * X, int ld, int kb, lkb_pf_act a, int rows, lkb_stream_t st);
/* ref: src/prefill.cuh:108  k_pf_swiglu */
int lkb_pf_swiglu(const float * Y, int ld, int up_off, int kb, lkb_pf_act a, int rows, lkb_stream_t st);
/* ref: src/prefill.cuh:109-114  k_pf_router / k_pf_router_small.  The engine
 * picks the small form for m <= 256 (ref: src/engine.cu:1170-1176); so does this. */
int lkb_pf_router(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                  float * sel, float * sig, lkb_stream_t st);
/* The tiled form for any m (what lkb_pf_router picks above 256 tokens).  A caller that splits one chunk
 * over several GPUs uses it to keep the form -- and with it every logit bit -- independent of the split. */
int lkb_pf_router_tiled(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, lkb_stream_t st);
int lkb_pf_router_small(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, lkb_stream_t st);
/* ref: src/prefill.cuh:115-116  k_pf_select */
int lkb_pf_select(const float * sel, const float * sig, int m, int * idx, float * w, lkb_stream_t st);
/* lkb_pf_router_small (small_form != 0) or lkb_pf_router_tiled followed by lkb_pf_select, in ONE launch: the CTA that
 * produced a token's 64 sel / sig values selects its top-4 from shared memory (sel / sig are still written).  Same
 * results as the two calls.  No counterpart in the reference (its engine launches the two kernels, src/engine.cu:1170-1180). */
int lkb_pf_router_select(const float * H, int m, int small_form, const float * Wr, const float * bias, const float * inv,
                         float * sel, float * sig, int * idx, float * w, lkb_stream_t st);
/* ref: src/prefill.cuh:117-122  k_pf_moe_count / _plan / _scatter.  cnt must be
 * zero on entry to count (the engine memsets it, ref: src/engine.cu:1182). */
int lkb_pf_moe_count(const int * idx, int n, int * cnt, lkb_stream_t st);
/* ref: src/engine.cu:1182  cudaMemsetAsync(p.cnt, 0, 64*4, st) -- the zeroing that precedes the count */
int lkb_zero_i32(int * p, int n, lkb_stream_t st);
int lkb_pf_moe_plan(const int * cnt, int * off, int * tiles, int * ntiles, lkb_stream_t st);
int lkb_pf_moe_scatter(const int * idx, int n, const int * off, int * perm, lkb_stream_t st);
/* ref: src/prefill.cuh:69-71  pf_gemm_dense / pf_gemm_moe / pf_gemm_swiglu */
int lkb_pf_gemm_dense(const lkb_pf_gemm * g, lkb_stream_t st);
int lkb_pf_gemm_moe(const lkb_pf_gemm * g, int max_tiles, lkb_stream_t st);
int lkb_pf_gemm_swiglu(const lkb_pf_gemm * g, int max_tiles, lkb_stream_t st);
/* Kernel-configuration selector of the three launchers above: -1 (default) the
 * tensor-core form wherever it covers the shape, 0 the CUDA-core form, 1 the
 * tensor-core form or an error.  Also read once from the environment variable
 * LKB_PF_CFG by lkb_init().  ref: src/prefill.cu:813-848 (LK_PF_CFG_DENSE/MOE/SWIGLU) */
int lkb_pf_gemm_config(int cfg);
/* Per-block term of the three launchers above.  1 (default): the reference's shipped form -- the block sum
 * arrives as the float 12582912 + S_b and the offset is folded into c = fma(d8, 12582912, 8sum):
 * acc = fma(d4, fma(d8, 12582912 + S_b, -c), acc); fp32 results are bit-identical to the reference's kernel and
 * within its own gate of float64 (half an ulp of c per block).  0: the exact term of the decode kernels,
 * acc = fma(d4, fma(d8, float(S_b), -8sum), acc), within 1e-5 of float64 at one more packed add per value pair.
 * The int32 block sums S_b are exact either way.  Also read once from LKB_PF_ARITH by lkb_init().
 * ref: src/prefill.cu:131-139 (PF_EPI2), 341-342, 381-399 */
int lkb_pf_gemm_arith(int fold);
/* Optional workspace of the grouped (perm != NULL) tensor-core form.  With a workspace registered, lkb_pf_gemm_moe /
 * lkb_pf_gemm_swiglu first copy the activation rows into token-tile order (one small kernel) and the GEMM then fetches
 * every 128-token tile with one bulk tensor copy; without one the rows are gathered through perm inside the GEMM, four
 * per copy, which is slower.  Results are identical.  The buffer is the caller's (this library allocates nothing):
 * 256-byte aligned device memory of at least lkb_pf_gemm_workspace_bytes(max_tiles, K of the widest activation)
 * bytes; it is read and written by every grouped GEMM launched afterwards, so calls that share it must be ordered on
 * one stream.  ptr = NULL unregisters.  No counterpart in the reference (its kernel gathers rows with cp.async). */
int lkb_pf_gemm_workspace_bytes(int max_tiles, int k_max, size_t * bytes_out);
int lkb_pf_gemm_set_workspace(void * ptr, size_t bytes);
/* Every device-side wait of the tensor-core form is bounded; this SYNCHRONISES the device and
 * returns 0, or the code of the first wait that expired since the last call (10 producer,
 * 15 expansion, 20/21 MMA issuer, 30/31 epilogue) and clears it.  No counterpart in the reference. */
int lkb_pf_gemm_status(void);
/* ref: src/prefill.cuh:123-127  k_pf_moe_combine / k_pf_moe_combine_norm / k_pf_pack_q8_1 */
int lkb_pf_moe_combine(float * X, const float * D, const float * w, int m, lkb_stream_t st);
int lkb_pf_moe_combine_norm(float * X, const float * D, const float * w, const float * nw, lkb_pf_act a,
                            float * inv_out, int m, lkb_stream_t st);
int lkb_pf_pack_q8_1(lkb_pf_act a, int t, lkb_block_q8_1 * y, lkb_stream_t st);

/* ------------------------------------------------ expert-parallel dispatch */
/* Helpers of the multi-GPU prefill; no counterpart in the reference (single GPU).  A slot's activation
 * travels as one LKB_EP_ROW_BYTES row: 2048 B quants | 512 B (d8, 8sum) | 1/rms | expert id on the owner.
 * pack: row p = slot send_order[p] (token = slot >> 2), pos[slot] = p.  unpack: rows -> planar Q8_1 + inv +
 * local expert ids.  combine_norm_gather: lkb_pf_moe_combine_norm with the D row of slot s at D[pos[s]]. */
#define LKB_EP_ROW_BYTES (LKB_HIDDEN + (LKB_HIDDEN / 32) * 8 + 16)
int lkb_ep_pack_rows(lkb_pf_act a, const float * inv, const int * idx, const int * send_order, int n,
                     int experts_per_rank, void * out, int * pos, lkb_stream_t st);
int lkb_ep_unpack_rows(const void * in, int n, lkb_pf_act a, float * inv, int * local_expert, lkb_stream_t st);
int lkb_pf_moe_combine_norm_gather(float * X, const float * D, const int * pos, const float * w, const float * nw,
                                   lkb_pf_act a, float * inv_out, int m, lkb_stream_t st);

/* ---- output projection (Q6_K), argmax, embedding row ----------------------------------------------
 * Q6_K planes as the reference lays them out: per 256-element super-block ql[128] (low nibbles), qh[64]
 * (2 high bits), sc[16] (int8 sub-block scales) and one fp16 d.  ref: src/quant.cuh:171-250
 *
 * lkb_gemv_q6_K: y[r] = ninv * sum over row r of Q6_K weight x Q8_1 activation, in the shipped integer form
 * (lane L owns elements 8L..8L+7 of every super-block; one fp32 term per lane and super-block; xor butterfly).
 * ssq != NULL folds the producer's 1/rms (lkb_norm_produce) into the result; NULL means ninv = 1.
 * sbpr = super-blocks per row (K / 256).  sbpr == 8 with 16-byte aligned planes takes the streaming kernel,
 * anything else a plain warp-per-row kernel with the same arithmetic.
 * ref: src/kernels.cu:426-478 (k_gemv_q6_K_dp4a), src/kernels.cu:359 (k_gemv_q6_K, same arguments) */
int lkb_gemv_q6_K(const void * ql, const void * qh, const void * sc, const void * d, const lkb_block_q8_1 * xq,
                  int out_rows, int sbpr, float * y, const float * ssq, float eps, lkb_stream_t st);
/* Bounded-wait status of the streaming kernel: 0, or the code of the wait that gave up (then cleared).
 * No counterpart in the reference. */
int lkb_gemv_q6_K_status(void);
/* Two-stage argmax, lowest index among equal maxima.  Stage 1 writes ceil(n / 1024) partial (value, index)
 * pairs; stage 2 reduces n partials, stores the token id and, when d_pos is non-null, adds 1 to it (the
 * reference advances its device-side position in the same kernel).  ref: src/kernels.cu:954-995 */
int lkb_argmax_part(const float * v, int n, float * pv, int * pi, lkb_stream_t st);
int lkb_argmax_final(const float * pv, const int * pi, int n, int * d_token, int * d_pos, lkb_stream_t st);
/* x[0..n) = dequantised row *d_token of a Q6_K matrix with n columns (n % 256 == 0).
 * ref: src/kernels.cu:855-868 (k_embed_q6_K), src/quant.cuh:171-190 */
int lkb_embed_q6_K(const void * ql, const void * qh, const void * sc, const void * d, const int * d_token, int n,
                   float * x, lkb_stream_t st);

/* ---- sequence mixers of a decode step -----------------------------------------------------------------
 * Model constants of the attention kernels: 32 query heads, 8 KV heads, head_dim 64; fp16 KV cache laid out
 * [position][kv_head][64].  ref: src/kernels.cuh:14-24 */
#define LKB_ATTN_SPLIT 18                 /* slices per KV head (partial-buffer stride) */
#define LKB_ATTN_PARTW 66                 /* floats per partial: running max, sum, 64 accumulators */
/* Split-K decode attention over positions 0..*d_pos.  part = float[32][LKB_ATTN_SPLIT][LKB_ATTN_PARTW];
 * lkb_attn_combine merges the live slices, writes out[32*64] (may be NULL) and the Q8_1 form of it (yq8,
 * 64 blocks, may be NULL).  The float64 evaluation is the definition (ref: tests/test_attn.cu:46-75); the
 * slice rule differs from the reference's (here ceil(seq/256) slices, at most 18, whole 32-token groups).
 * ref: src/kernels.cu:1303-1560 (k_attn_split), src/kernels.cu:1562-1599 (k_attn_combine) */
int lkb_attn_split(const float * q, const void * kc, const void * vc, const int * d_pos, float * part, lkb_stream_t st);
int lkb_attn_combine(const float * part, const int * d_pos, float * out, lkb_block_q8_1 * yq8, lkb_stream_t st);
/* Per-head RMSNorm (eps 1e-5) with weights qn / kn, NEOX half-split RoPE at position *d_pos, in place on
 * qf[32*64] and kf[8*64]; appends the rotated K and vf[8*64] as fp16 to the cache row *d_pos.  theta is the
 * RoPE base (the reference compiles in 1e7).  ref: src/kernels.cu:871-915 (k_qk_norm_rope) */
int lkb_qk_norm_rope(float * qf, float * kf, const float * vf, const float * qn, const float * kn, const int * d_pos,
                     void * kc, void * vc, float theta, lkb_stream_t st);
/* One decode step of the short gated convolution over n channels: bcx = [B | C | X], conv_w[ch*3 + tap],
 * hist[ch*2 + {0,1}] (updated in place), y = C * (h0*w0 + h1*w1 + (B*X)*w2) as fp32 (may be NULL) and as
 * Q8_1 blocks (may be NULL).  t is unused, as in the reference.  ref: src/kernels.cu:521-545 (k_shortconv) */
int lkb_shortconv(const float * bcx, int t, const float * conv_w, float * hist, float * y, lkb_block_q8_1 * yq8, int n,
                  lkb_stream_t st);

/* ---- sequence mixers of batched prefill (a chunk of m tokens at positions P .. P+m-1) -------------------
 * With lkb_pf_gemm_dense for the in / out / q|k|v / output projections they complete a full-model prefill
 * chunk.  The per-token kernels evaluate their decode twins' arithmetic: a chunk leaves the same conv history,
 * KV rows and activations as m decode steps.
 * lkb_pf_embed: x[t][0..n) = dequantised Q6_K row toks[t].                         ref: src/prefill.cu:856-868
 * lkb_pf_conv: Y = in_proj output [m][6144] (B | C | X); planar Q8_1 rows of C * conv into a; hist is read.
 * lkb_pf_conv_hist: the two-tap history after the chunk (run after lkb_pf_conv).   ref: src/prefill.cu:937-970
 * lkb_pf_qknr: Y = q|k|v output [m][3072]; per-head RMSNorm + NEOX RoPE (base theta; the reference compiles in
 *   1e7); Q leaves as fp16 [m][2048] pre-scaled by 1/8, K and V are appended to the cache.  ref: src/prefill.cu:975-1016
 * lkb_pf_attn: causal GQA attention of the chunk's queries qh over cache positions 0 .. P+m-1, o = fp32 [m][2048].
 *   Definition: float64 softmax over the fp16 inputs; P is rounded to fp16 before the P V product, as in the
 *   reference (gate 4e-3 absolute, ref: tests/test_prefill.cu:244-289).              ref: src/prefill.cu:1029-1268 */
int lkb_pf_embed(const void * ql, const void * qh, const void * sc, const void * d, const int * toks, float * x, int n, int m,
                 lkb_stream_t st);
int lkb_pf_conv(const float * Y, const float * cw, const float * hist, lkb_pf_act a, int m, lkb_stream_t st);
int lkb_pf_conv_hist(const float * Y, int m, float * hist, lkb_stream_t st);
int lkb_pf_qknr(const float * Y, const float * qn, const float * kn, int P, void * qh, void * kc, void * vc, int m, float theta,
                lkb_stream_t st);
int lkb_pf_attn(const void * qh, int m, int P, const void * kc, const void * vc, float * o, lkb_stream_t st);

/* ---- expert-parallel prefill over NVLink peer memory (no host round trip, no NCCL on the data path) ----------------
 * No counterpart in the reference (it is single-GPU).  Every rank owns four buffers in symmetric memory, mapped into
 * every peer; lkb_ep_peers holds the G peer views of each (index = rank, own rank included):
 *   cmat   int[G*G]            count matrix, row s = rows rank s sends to each rank
 *   flags  int[3*8]            arrival flags (phase 0 counts, 1 dispatched rows, 2 returned rows) per source rank
 *   recv   byte[cap][2576]     dispatched rows (LKB_EP_ROW_BYTES each), cap = worst case = every slot of the chunk
 *   dback  float[slots][2048]  this rank's D rows, in its send order
 * epoch is a device int the caller zeroes once: lkb_ep_route_exchange advances it by one per layer and the other
 * kernels read it (flags are never reset, and nothing on the host changes from layer to layer); status (device int,
 * 0 = fine) receives a code when a bounded wait expires: 1 counts, 2 / 3 / 4 = the wait of phase 0 / 1 / 2.  A wait
 * lasts at most the limit set by lkb_ep_set_wait_limit_ms (default 5000 ms; 1..60000); once a code is recorded the
 * later waits return at once.
 * lkb_ep_route_exchange leaves offs[3*G+1] (send bases, receive offsets, return bases, rows received).
 * lkb_ep_pack_push: row p of my send order -> its owner's recv buffer; doff[g] = first position of destination g in
 * my send order; pos[slot] = p. */
typedef struct {
    void * cmat[8];
    void * flags[8];
    void * recv[8];
    void * dback[8];
} lkb_ep_peers;
/* No counterpart in the reference: the exchange over peer memory described above. */
int lkb_ep_set_wait_limit_ms(int ms);
/* No counterpart in the reference: dispatch, arrival wait and return of the exchange described above. */
int lkb_ep_pack_push(lkb_pf_act a, const float * inv, const int * idx, const int * send_order, const int * doff, const int * offs,
                     int n, int experts_per_rank, const lkb_ep_peers * peers, int me, int G, const int * epoch, int * pos, unsigned * done,
                     lkb_stream_t st);
int lkb_ep_wait(const int * flags, int phase, int G, const int * epoch, int * status, lkb_stream_t st);
/* No counterpart in the reference: the home side's routing and count exchange in ONE launch -- slots grouped by the
 * rank owning their expert (send_order[n], doff[64]: first position of each destination; stable, the order of
 * lkb_pf_moe_count / _plan / _scatter keyed by owner rank), then the count exchange: my count row into every rank's
 * matrix, flags, wait for all rows, offsets.  One CTA; n is a rank's slots of a chunk (a few thousand). */
int lkb_ep_route_exchange(const int * idx, int n, int experts_per_rank, const lkb_ep_peers * peers, int me, int G, int * epoch,
                          int * send_order, int * doff, int * offs, int * status, lkb_stream_t st);
/* No counterpart in the reference: the owner side's wait for the dispatched rows (lkb_ep_wait phase 1) and the grouped
 * GEMM's plan over them (cnt[64], off[64], tiles, ntiles, perm: the results of lkb_pf_moe_count / _plan / _scatter
 * keyed by the local expert id each received row carries, with the row count read from device memory) in ONE launch.  nrecv_out (optional) receives
 * the row count.  When the wait gives up, *ntiles = 0 and the status word holds the code. */
int lkb_ep_route_experts(const void * recv, int cap, const int * flags, int G, const int * epoch, const int * offs, int * cnt, int * off,
                         int * tiles, int * ntiles, int * perm, int * nrecv_out, const lkb_ep_peers * peers, float ** home_rows,
                         float * inv_out, int * status, lkb_stream_t st);
/* No counterpart in the reference.  home_rows (optional, with peers) of lkb_ep_route_experts receives, per received
 * row, the address its result row has in its home rank's return buffer; lkb_pf_gemm_moe_rows is lkb_pf_gemm_moe
 * writing the output row of slot s to out_rows[s] instead of out + s * out_ld (plain stores, peer memory included;
 * add must be 0; tensor-core form only, else LKB_ERR_UNSUPPORTED), so the down projection's rows travel home while
 * the GEMM still computes; lkb_ep_publish_wait then announces phase 2 of the epoch to every rank. */
int lkb_pf_gemm_moe_rows(const lkb_pf_gemm * g, int max_tiles, float * const * out_rows, lkb_stream_t st);
/* No counterpart in the reference.  inv_out (optional) of lkb_ep_route_experts receives the received rows' 1/rms as a
 * plane; lkb_pf_gemm_swiglu_packed is lkb_pf_gemm_swiglu reading its activations from PACKED rows of row_pitch bytes
 * (bpr*32 quants, then bpr (d8, 8sum) pairs; g->aqs = the first row, g->asc unused) -- the dispatch rows as they
 * arrived, so no unpack pass is needed.  Needs the registered workspace (the row gather reads the packed rows);
 * tensor-core form only. */
int lkb_pf_gemm_swiglu_packed(const lkb_pf_gemm * g, int max_tiles, int row_pitch, lkb_stream_t st);
/* Publish `phase` of the epoch to every rank, then wait for the same phase of every source (lkb_ep_wait), in one
 * launch.  No counterpart in the reference. */
int lkb_ep_publish_wait(const lkb_ep_peers * peers, int me, int G, int phase, const int * epoch, const int * flags, int * status,
                        lkb_stream_t st);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* LKB_H */
