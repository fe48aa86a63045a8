/* seedless_b200.h -- C ABI of libseedless_b200.so
 *
 * A B200 (sm_100a) implementation of the Seedless decode core of penta2himajin/qwisp: the
 * per-token forward of a Qwen3-hybrid MoE model with 4-bit MLX-affine group-64 weights.
 * The reference exposes this path as a Swift struct of closures that its Tell runtime calls
 * (`Tell.SpecBackend`, swift/Sources/QwispCore/TellRuntime.swift:83-111) plus the batched
 * engine protocol `BatchSlots` (swift/Sources/QwispCore/ContinuousBatch.swift:38-66); each
 * entry point below names the closure / method it replaces.
 *
 * Conventions: every function returns an int32 status, 0 = ok, < 0 = error.  After any
 * device-side or injected failure the engine is poisoned: every later call on it returns
 * SL_ERR_POISONED and sl_last_fault() returns the first fault's text (the reference's GPU
 * fault firewall, swift/Sources/QwispCore/SeedlessFusedVerify.swift:376-416).
 * One thread at a time per engine (the reference serialises decode the same way,
 * swift/Sources/QwispCore/LLMBackend.swift:121-142).  All pointers are plain host pointers
 * unless a parameter says "device".  fp16 values are passed as uint16_t bit patterns.
 * There is no CPU fallback: every entry point fails with SL_ERR_NO_DEVICE without a GPU.
 */
#ifndef SEEDLESS_B200_H
#define SEEDLESS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    SL_OK = 0,
    SL_ERR_INVALID = -1,      /* bad argument / shape */
    SL_ERR_NO_DEVICE = -2,    /* no usable CUDA device */
    SL_ERR_CUDA = -3,         /* a CUDA call failed (engine poisoned) */
    SL_ERR_POISONED = -4,     /* engine already poisoned by an earlier fault */
    SL_ERR_CAPACITY = -5,     /* rows > max_rows, sequence > max_seq_len, out of KV pages ... */
    SL_ERR_NOT_FOUND = -6,    /* unknown tensor name */
    SL_ERR_FORMAT = -7        /* malformed state blob */
};

/* Model geometry (swift/Sources/QwispCore/QwispModel.swift:83-120; the reference hard-codes
 * these, swift/Sources/QwispCore/SeedlessEngine.swift:13-16) and engine sizing
 * (maxM / maxSeqLen of SeedlessFusedForward.init, SeedlessFusedVerify.swift:3368-3374).
 * Fixed by the kernels: GDN head dim 128, conv kernel 4, attention head dim 256, rope dim 64,
 * group size 64, 4 bit.  hidden and moe_inter must be multiples of 256. */
typedef struct sl_config {
    int32_t hidden;          /* 2048 */
    int32_t n_layers;        /* 40 */
    int32_t attn_every;      /* 4: layer i is full attention iff (i+1) % attn_every == 0 */
    int32_t vocab;           /* 151936 (multiple of 16) */
    int32_t n_experts;       /* 256 (<= 256) */
    int32_t top_k;           /* 8 */
    int32_t moe_inter;       /* 512 */
    int32_t gdn_k_heads;     /* 16 */
    int32_t gdn_v_heads;     /* 32 */
    int32_t attn_heads;      /* 16 */
    int32_t attn_kv_heads;   /* 2 */
    float rope_theta;        /* 1e7 */
    float rms_eps;           /* 1e-6 */
    int32_t max_rows;        /* rows (tokens) per call, all streams together */
    int32_t max_streams;     /* stream slots (each holds GDN state + a KV page table) */
    int32_t kv_page_size;    /* positions per KV page (multiple of 32) */
    int32_t kv_pages;        /* pages in the engine's KV arena, shared by all streams */
    int32_t flags;           /* SL_FLAG_* bits, 0 = defaults (how the step is assembled; results do not depend on them) */
} sl_config;

/* sl_config.flags: assembly switches for measurements and debugging.  Every combination gives the same tokens. */
enum {
    SL_FLAG_NO_GRAPH = 1,          /* launch every kernel of a decode step eagerly instead of replaying a CUDA graph */
    SL_FLAG_NO_PDL = 2,            /* no programmatic dependent launch between the kernels of a step */
    SL_FLAG_STEP_KERNEL = 4,       /* single-stream decode steps as ONE cooperative kernel launch (see sl_engine_use_persistent) */
    SL_FLAG_SPLIT_EXPERTS = 8,     /* batch-1 decode: gate/up and down as two launches instead of the fused expert kernel */
    SL_FLAG_ROUTE_IN_ROUTER = 16,  /* batch-1 decode: the router kernel's last CTA routes (instead of every CTA of the expert kernel) */
    SL_FLAG_L2_PREFETCH = 32,      /* kernels prefetch the weights of later kernels into L2 (slower as measured; kept for comparison) */
    SL_FLAG_PASS_KERNELS = 64      /* calls with more than 8 rows walk them in passes of 8 with the one-to-eight-row kernels instead of the many-row kernels (same bits) */
};

/* One named tensor handed to sl_engine_create.  Names: "embed", "final_norm", "lm_head.w/.s/.b",
 * "L<i>.in_norm", "L<i>.post_norm", "L<i>.gdn.in_proj_qkv.w/.s/.b" (also _z,_b,_a),
 * "L<i>.gdn.conv_w" (f32 [convDim,4]), "L<i>.gdn.A_log", "L<i>.gdn.dt_bias" (f32),
 * "L<i>.gdn.norm", "L<i>.gdn.out_proj.*", "L<i>.attn.q_proj.*" (k_,v_,o_), "L<i>.attn.q_norm",
 * "L<i>.attn.k_norm", "L<i>.moe.router" (fp16 [E,H]), "L<i>.moe.shared_gate" (fp16 [H]),
 * "L<i>.moe.gate_proj.*" ([E*I,H]), "L<i>.moe.up_proj.*", "L<i>.moe.down_proj.*" ([E*H,I]),
 * "L<i>.moe.shared_gate_proj.*", "L<i>.moe.shared_up_proj.*", "L<i>.moe.shared_down_proj.*".
 * 4-bit tensors are in the MLX affine layout: .w uint32 [N,K/8] (8 nibbles per word, low
 * first), .s/.b fp16 [N,K/64] (SeedlessMetalForward.swift:219-221).  The data is copied.
 * "embed" may instead be given as the checkpoint's 4-bit table "embed.w/.s/.b" ([vocab,hidden]);
 * it is expanded once into the fp16 table with the reference's per-row arithmetic
 * (embed_rows_q4, SeedlessFusedVerify.swift:556-570), so lookups give the same halves.
 * "L<i>.moe.router" and "L<i>.moe.shared_gate" may instead be given, per layer, in the checkpoint's
 * 8-bit group-64 layout: "L<i>.moe.router.w" (bytes [E,H]), ".s/.b" (fp16 [E,H/64]),
 * "L<i>.moe.shared_gate.w" (bytes [H]), ".s/.b" (fp16 [H/64]) - all six or none; the router kernel then
 * runs the reference's 8-bit GEMV arithmetic (qmm8, SeedlessMetalForward.swift:384-434).
 * "L<i>.gdn.norm.f32" (f32 [128]) may replace "L<i>.gdn.norm": that layer's gated norm then keeps the
 * normed value in f32, the reference's behaviour for an f32 weight (SeedlessFusedVerify.swift:2815-2818). */
typedef struct sl_weight_desc {
    const char* name;
    const void* data;
    uint64_t nbytes;
    int32_t on_device;       /* 0 = host pointer, 1 = device pointer */
} sl_weight_desc;

/* Seeded synthetic weights generated on the device (integer hash -> Irwin-Hall normal ->
 * fp16 -> 4-bit affine quantiser), bit-identical to the CPU oracle's generator. */
typedef struct sl_synth_spec {
    uint64_t seed;
    float norm_jitter;       /* RMSNorm weights = 1 + N(0, norm_jitter); 0 => exactly 1 */
    float conv_std;          /* std of the depthwise conv weights */
} sl_synth_spec;

typedef struct sl_engine sl_engine;
typedef struct sl_stream sl_stream;
typedef struct sl_fullsnap sl_fullsnap;
typedef struct sl_snap { int32_t kv_len; int32_t parity; int32_t valid; int32_t calls; } sl_snap;

/* ---- engine (SeedlessEngine.build + makeFused, SeedlessEngine.swift:33-144) ---- */
int32_t sl_engine_create(const sl_config* cfg, const sl_weight_desc* weights, int32_t n_weights, sl_engine** out);
int32_t sl_engine_create_synthetic(const sl_config* cfg, const sl_synth_spec* synth, sl_engine** out);
int32_t sl_engine_destroy(sl_engine* e);
/* Run all work of this engine on the given CUDA stream (a cudaStream_t); NULL = the engine's own. */
int32_t sl_engine_set_cuda_stream(sl_engine* e, void* cuda_stream);
/* Copy a named tensor back to the host (parity checks of the loader / generator). */
int32_t sl_engine_read_tensor(sl_engine* e, const char* name, void* host_buf, uint64_t nbytes);
int32_t sl_engine_tensor_bytes(sl_engine* e, const char* name, uint64_t* nbytes);
/* Sticky fault text or NULL (SpecBackend.gpuFault, TellRuntime.swift:107-110). */
const char* sl_last_fault(sl_engine* e);
/* Host-side test hook: the next device-touching call reports failure and poisons the engine
 * (mirrors `injectCBFailure`, SeedlessFusedVerify.swift:403-404).  Never faults the GPU. */
int32_t sl_inject_fault(sl_engine* e, int32_t on);
/* Test hook for the device-side half of the fault firewall: enqueues a one-CTA kernel whose bounded wait
 * (the routine the weight stages use, limited to a thousand polls on a barrier nothing arms) runs out and
 * reports through the engine's error word.  Nothing faults or hangs.  The next call that synchronises
 * returns SL_ERR_CUDA and poisons the engine, as it does when a real kernel's wait gives up. */
int32_t sl_debug_wait_timeout(sl_engine* e);
/* Kernels this library has launched so far (bench bookkeeping). */
int64_t sl_engine_launch_count(sl_engine* e);
/* Replay decode steps as CUDA graphs (default on) or launch every kernel eagerly. */
int32_t sl_engine_use_graphs(sl_engine* e, int32_t on);
/* Single-stream decode steps (sl_step_argmax with one row, chained steps) run as the kernel-per-phase assembly
 * that serves every other call (the default: it is the faster one on B200 as measured), or as ONE cooperative
 * kernel launch per token when the geometry and the device allow it.  Both produce the same tokens and leave the
 * same caches.  on = 0 / 1 selects; on < 0 only queries.  Returns 1 when the one-kernel step is available
 * (query: and selected), 0 otherwise.  SL_FLAG_STEP_KERNEL in sl_config.flags selects it at creation. */
int32_t sl_engine_use_persistent(sl_engine* e, int32_t on);
/* Profiling of the one-kernel step: on = 1 arms a timeline (returns the number of CTAs); every following step
 * overwrites it with nanosecond stamps of each CTA's phase boundaries, [CTA][layer + 1][24] uint32 relative to the
 * CTA's start; on = 0 disarms it and, when out is given, copies the last step's stamps to the host. */
int32_t sl_debug_step_timeline(sl_engine* e, int32_t on, uint32_t* out, uint64_t cap_words);
/* Per-kernel timing with CUDA events on the launching stream, for eager launches only (the
 * reference's profiled forward splits its command buffer per stage for the same purpose,
 * SeedlessFusedVerify.swift:4352-4378).  The report has one line per kernel:
 * "name launches total_ms algorithmic_bytes". */
int32_t sl_profile_start(sl_engine* e);
int32_t sl_profile_report(sl_engine* e, char* buf, uint64_t cap);

/* ---- stream = one sequence's caches: KV page table + GDN state ("backend instance" /
 *      "lane", SeedlessFusedVerify.swift:3368-3452, LaneServe.swift:256) ---- */
int32_t sl_stream_create(sl_engine* e, int32_t max_seq_len, sl_stream** out);
int32_t sl_stream_destroy(sl_stream* s);
int32_t sl_stream_len(sl_stream* s);
int32_t sl_stream_reset(sl_stream* s);

/* SpecBackend.forward (TellRuntime.swift:84; SeedlessFusedVerify.swift:3641): embed + all
 * layers + final norm for M tokens appended at the current position; out_normed_f16 [M,H]
 * (may be NULL). */
int32_t sl_forward(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_normed_f16);
/* SpecBackend.forwardHybrid (TellRuntime.swift:96-99; SeedlessFusedVerify.swift:4215-4345): the
 * prefill-only forward.  Same contract and outputs as sl_forward, but the dense projections and the experts run
 * as tcgen05 tensor-core GEMMs on dequantised fp16 weights, the router logits and attention on tensor-core tiles.
 * As in the reference the result is NOT bit-identical to sl_forward (f32 summation orders differ) but it is
 * deterministic and independent of how a prompt is split into calls, down to one-row pieces.  Which family runs
 * is decided by which entry point is called, never by M. */
int32_t sl_forward_hybrid(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_normed_f16);
/* SpecBackend.hybridChunk (TellRuntime.swift:234-238): rows per prefill call = min(1024, max_rows). */
int32_t sl_hybrid_chunk(sl_engine* e);
/* SpecBackend.stepArgmax (SeedlessFusedVerify.swift:3832-3912): forward + lm_head + per-row
 * greedy argmax (first maximum wins); only int32[M] is read back. */
int32_t sl_step_argmax(sl_stream* s, const int32_t* tokens, int32_t M, int32_t* out_tokens);
/* SpecBackend.chainedStepArgmax (SeedlessFusedVerify.swift:4405-4513): K greedy steps with
 * the token fed back on the device; identical to K calls of sl_step_argmax with M = 1. */
int32_t sl_chained_step_argmax(sl_stream* s, int32_t first, int32_t K, int32_t* out_tokens);
/* The same split in two so a caller can time the device work alone: enqueue K chained steps
 * (first < 0: continue from the token the previous step produced, already on the device),
 * then collect the K tokens (synchronises). */
int32_t sl_chained_enqueue(sl_stream* s, int32_t first, int32_t K);
int32_t sl_chained_collect(sl_stream* s, int32_t K, int32_t* out_tokens);
/* SpecBackend.stepLogitsRows (TellRuntime.swift:115-121): full fp16 logits [M,V] read back. */
int32_t sl_step_logits(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_logits_f16);

/* SpecBackend.snapshot / rollback (SeedlessFusedVerify.swift:4039-4047): undo exactly one
 * following forward/step: KV length rewind + GDN ping-pong swap.  The snapshot remembers the stream's
 * call count; a rollback after anything but exactly one call (each chained step counts) is refused
 * with SL_ERR_INVALID. */
int32_t sl_snapshot(sl_stream* s, sl_snap* out);
int32_t sl_rollback_one_step(sl_stream* s, const sl_snap* snap);
/* fullSnapshot / fullRestore (SeedlessFusedVerify.swift:4053-4068): arbitrary rewind inside
 * the same stream: KV length + deep copy of the GDN state. */
int32_t sl_full_snapshot(sl_stream* s, sl_fullsnap** out);
int32_t sl_full_restore(sl_stream* s, const sl_fullsnap* snap);
int32_t sl_fullsnap_free(sl_fullsnap* snap);
/* persistentStateData / restorePersistentState (SeedlessFusedVerify.swift:4077-4154): the
 * self-describing "QWS1" blob; restorable into a stream of a different max_seq_len.
 * sl_state_restore returns SL_ERR_FORMAT on any mismatch; the stream must then be reset. */
int32_t sl_state_size(sl_stream* s, uint64_t* nbytes);
int32_t sl_state_save(sl_stream* s, void* buf, uint64_t nbytes);
int32_t sl_state_restore(sl_stream* s, const void* buf, uint64_t nbytes);

/* BatchSlots.step / SeedlessLaneBatch.stepArgmaxBatch (SeedlessLaneBatch.swift:876): one
 * greedy step over B streams, one token each; row b is bit-identical to a solo step. */
int32_t sl_batch_step_argmax(sl_engine* e, sl_stream* const* streams, const int32_t* tokens, int32_t B, int32_t* out_tokens);

/* ---- speculative sampling on the device (stepSampleRows, SeedlessFusedVerify.swift:3954; kernel
 *      spec_sample_rows, SamplerGPU.swift:39-156) ----
 * Forward M rows, then per row: out_full = categorical draw by Gumbel-max at temperature 1/inv_temperature
 * over the top_p nucleus (top_p >= 0.999: whole vocabulary), out_resid = the same draw with
 * draft_tokens[m] excluded (= out_full when the draft is -1 or draft_tokens is NULL), out_accept = 1 when
 * coin < p(draft).  inv_temperature <= 0 is greedy: out_full equals sl_step_argmax's token.  The noise is a
 * counter-based hash of (seed_lo, seed_hi ^ (base_pos + m), token), so a call is reproducible.  Only the
 * three int32 arrays leave the device.
 * logit_adj: host f32 [vocab] or NULL: penalties + bias added to every row's logits before the maximum,
 * the nucleus, the draws and p(draft) are taken (the reference's logitAdj / LADJ, SamplerGPU.swift:41,69).
 * draft_tokens outside [-1, vocab) are refused with SL_ERR_INVALID before anything is launched. */
int32_t sl_step_sample_rows(sl_stream* s, const int32_t* tokens, int32_t M, const int32_t* draft_tokens, const float* logit_adj, float inv_temperature, float top_p,
                            uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, int32_t* out_full, int32_t* out_resid, int32_t* out_accept);
/* The sampling kernel alone on host logits [M, vocab] fp16 (kernel tests). */
int32_t sl_op_sample_rows(sl_engine* e, const uint16_t* logits_f16, int32_t M, const int32_t* draft_tokens, const float* logit_adj, float inv_temperature, float top_p,
                          uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, int32_t* out_full, int32_t* out_resid, int32_t* out_accept);

/* ---- expert-parallel batched decode (NO COUNTERPART IN THE REFERENCE, which runs on one GPU) ----
 * One process per GPU, each with its own engine holding the full model; rank r of `world` computes
 * experts [r*E/world, (r+1)*E/world) for the rows of every rank.  After sl_ep_init, a call of
 * sl_batch_step_argmax with exactly rows_per_rank streams runs the expert-parallel step: per MoE
 * layer an NCCL all-gather of the normed rows and routing indices, the local experts on all rows
 * that chose them, and an NCCL reduce-scatter of the pair outputs back to the rows' owners, who
 * combine them in ascending k.  All ranks must make that call in lockstep with the same row count.
 * Token streams are bit-identical to the single-GPU engine's.  cfg.max_rows must be at least
 * world * rows_per_rank.  Every other entry point (prefill, single steps) stays rank-local.
 * NCCL is resolved at run time from libnccl.so.2 (SL_ERR_NOT_FOUND if absent). */
int32_t sl_ep_unique_id(uint8_t* out128);                 /* rank 0: make the 128-byte id, share it by any host channel */
int32_t sl_ep_init(sl_engine* e, int32_t rank, int32_t world, const uint8_t* id128, int32_t rows_per_rank);

/* ---- single operators (the reference's per-op wrappers used by its kernel tests:
 *      SeedlessMetalForward.qmm SeedlessMetalForward.swift:222, routeTop8Rows
 *      SeedlessFusedVerify.swift:174, moeBlockRows / gdnLayerRows / attnLayerRows
 *      SeedlessVerifyForward.swift:37-248) ---- */
/* y[M,N] = x[M,K] . dequant4(W[N,K])^T; host buffers; N % 16 == 0, K in {256, 512, 1024, 2048, 4096}. */
int32_t sl_op_qmm4(const uint16_t* x_f16, const uint32_t* w, const uint16_t* scales_f16, const uint16_t* biases_f16,
                   int32_t M, int32_t K, int32_t N, uint16_t* y_f16);
/* The kernels read weights in a fragment-major layout made once at load time from the MLX layout:
 * wr holds (N/16) * (K/128) * 1024 bytes, sr holds (N/16) * (K/128) * 128 bytes (device buffers). */
int32_t sl_op_repack_q4_device(const void* w_dev, const void* s_dev, const void* b_dev, int32_t K, int32_t N,
                               void* wr_dev, void* sr_dev, void* cuda_stream);
/* The GEMV on device buffers in that layout, enqueued on cuda_stream without synchronising
 * (micro-benchmarks). */
int32_t sl_op_qmm4_device(const void* x_dev, const void* wr_dev, const void* sr_dev,
                          int32_t M, int32_t K, int32_t N, void* y_dev, void* cuda_stream);
/* The same product for MANY rows on the tcgen05 tensor cores (accumulator in tensor memory): the
 * GEMM form the reference uses for batched and prefill rows (tiled qmm, SeedlessMetalForward.swift:160-185).
 * Same buffers as sl_op_qmm4_device; N % 16 == 0.  Results agree with the GEMV form within fp16
 * rounding (every weight is dequantised to fp16 with one rounding and the whole K range accumulates in one f32 sum). */
int32_t sl_op_qmm4_tc_device(const void* x_dev, const void* wr_dev, const void* sr_dev,
                             int32_t M, int32_t K, int32_t N, void* y_dev, void* cuda_stream);
/* NO COUNTERPART IN THE REFERENCE.  Greedy tokens of final-normed rows x [M,K] against lm_head
 * weights in the fragment-major layout above: out_tokens_dev[m] = argmax_n (x[m] . dequant4(W[n])),
 * lowest n on ties, the same kernel sl_step_argmax ends with.  All pointers are device pointers;
 * the work is enqueued on cuda_stream and the call returns without synchronising.
 *
 * This entry point allocates nothing, at set-up or per call.  It is for hosts that cannot let a
 * library allocate: a serving process that has handed the whole of device memory to its own
 * arena at start-up (so a late allocation can fail, or steal pages the arena counts on), and
 * callers inside a latency-critical loop, where a device allocation may synchronise the whole
 * device and stall unrelated streams.  The per-CTA maxima and the completion counter the kernel
 * needs live in ONE fixed module-scope device array of 28,672 bytes, which bounds a call to
 * M <= 8 rows; a larger M returns SL_ERR_CAPACITY (with a line on stderr) and launches nothing.
 *   - The first call on each device looks up the array's address and sets the kernel's shared
 *     memory attribute; make that first call before starting a stream capture.
 *   - The array is shared by every caller in the process and keeps its last contents.  Only the
 *     counter must start at zero: each call clears it on cuda_stream ahead of the kernel, and
 *     the kernel leaves it at zero.  The maxima are overwritten before they are read.
 *   - Calls that overlap in time on the same device (two streams, two threads) race on the
 *     array and give undefined tokens: order them on one stream or with events. */
int32_t sl_op_lm_head_argmax_static(const void* x_dev, const void* wr_dev, const void* sr_dev,
                                    int32_t M, int32_t K, int32_t N, int32_t* out_tokens_dev, void* cuda_stream);
/* 4-bit affine quantiser on the device: w fp16 [N,K] -> packed/scales/biases (host buffers). */
int32_t sl_op_quantize_q4(const uint16_t* w_f16, int64_t N, int64_t K, uint32_t* packed, uint16_t* scales_f16, uint16_t* biases_f16);
/* MoE block of `layer` on already-normed rows x [M,H]: out [M,H], inds [M,top_k], scores fp16. */
int32_t sl_op_moe_block(sl_engine* e, int32_t layer, const uint16_t* x_f16, int32_t M,
                        uint16_t* out_f16, int32_t* inds, uint16_t* scores_f16);
/* Mixer (GDN or attention) of `layer` on already-normed rows x [M,H] placed at positions
 * pos0..pos0+M-1 of the stream; advances only that layer's cache, not the stream length. */
int32_t sl_op_mixer(sl_stream* s, int32_t layer, const uint16_t* x_f16, int32_t M, int32_t pos0, uint16_t* out_f16);
/* Test accessor: cached K (post-RoPE) and V of attention layer `layer` at positions pos0..pos0+n-1, each
 * as fp16 [kv_heads, n, 256] (either may be NULL); the positions must have been written (by a step or
 * by sl_op_mixer / sl_op_layer), whatever the stream's length says. */
int32_t sl_op_read_kv(sl_stream* s, int32_t layer, int32_t pos0, int32_t n, uint16_t* out_k_f16, uint16_t* out_v_f16);
/* One whole decoder layer (rmsnorm, mixer, +resid, rmsnorm, MoE, +resid; the reference's
 * decoder-layer test, SeedlessMetalForward.swift:3757) on residual-stream rows h_in [M,H] at
 * positions pos0..; advances only that layer's cache. */
int32_t sl_op_layer(sl_stream* s, int32_t layer, const uint16_t* h_in_f16, int32_t M, int32_t pos0, uint16_t* h_out_f16);
/* Head of the step on residual-stream rows: final norm + lm_head + greedy argmax. */
int32_t sl_op_head(sl_engine* e, const uint16_t* h_rows_f16, int32_t M, uint16_t* out_logits_f16, int32_t* out_tokens);
/* final-norm'ed rows -> logits (may be NULL) and greedy tokens (may be NULL). */
int32_t sl_op_lm_head(sl_engine* e, const uint16_t* normed_f16, int32_t M, uint16_t* out_logits_f16, int32_t* out_tokens);

/* ---- synthetic data helpers (same generator as the engine's weights) ---- */
int32_t sl_synth_tokens(uint64_t seed, const char* name, int64_t n, int32_t vocab, int32_t* out);
int32_t sl_synth_f16(uint64_t seed, const char* name, int64_t n, float mean, float std, uint16_t* out_f16);

#ifdef __cplusplus
}
#endif
#endif
