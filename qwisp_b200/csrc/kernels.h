// kernels.h -- argument blocks and host launchers of the Seedless B200 kernels.
#pragma once
#include "gemv.cuh"
#include <functional>

namespace sl {

struct Q4W { const uint32_t* w = nullptr; const __half* s = nullptr; const __half* b = nullptr; int64_t N = 0; int K = 0; };

struct DenseArgs {
    int lg_slices = 0;                   // log2(K/256), filled by the launcher
    unsigned* err = nullptr;             // set to 1 if a bounded wait on a bulk copy gave up
    __half* norm_scratch = nullptr;      // [M][K] scratch for the tensor-core path (normed rows); nullptr keeps the GEMV path
    bool tc = false;                     // prefill mode: dense projections on the tcgen05 GEMM (set per call by the caller)
    __half* xq = nullptr; float* sxq = nullptr;   // [M][K] / [M][K/64] scratch of the many-row kernels (calls with more than 8 rows); nullptr: pass kernels
    Q4R q;                                                       // repacked weights (tiles of 16 rows)
    int N, K, M;                                                 // N outputs (= 16 * tiles)
    const __half* x; int ldx;                                    // activations (plain) / residual stream (rmsnorm) / y (normgate)
    const __half* nw;                                            // norm weight
    const float* nw32 = nullptr;                                 // gated norm: f32 norm weight (norm in f32); nw keeps its fp16 cast
    const __half* z; int ldz;                                    // gate input of the gated norm
    float eps;
    __half* y; int ldy;                                          // output rows
    __half* logits;                                              // optional [M][N] (argmax epilogue)
    float* pval; int* pidx; int* out_tok; unsigned* counter;     // argmax partials / result / ticket
    PfList pf;                                                   // weights of later kernels to pull into L2
};

// what a kernel needs to raise this rank's flags at its peers (world == 0: not expert-parallel)
struct EpSignal { unsigned* flags[8]; unsigned* ctr; unsigned* ticket; int world = 0, rank = 0, layer = 0; };
// the router's dispatch: peer gather buffers + flags
struct EpDispatch { __half* pbuf[8]; int* ibuf[8]; EpSignal sig; };

struct MoeLists {
    int* n_active;       // [1]
    int* slot_expert;    // [E]
    int* slot_off;       // [E]
    int* slot_cnt;       // [E]
    int* pairs;          // [M*top_k] pair ids (row*top_k + k) grouped by expert slot
};

struct RouterArgs {
    const __half* h; int ldh;            // input rows
    const __half* norm_w; float eps;     // post-attention norm (nullptr: rows are already normed)
    const __half* router;                // fp16 [E][H]
    const __half* shared_gate;           // fp16 [H]
    // the checkpoint's 8-bit group-64 form of the two (set all six or none; they replace the fp16 pair)
    const uint8_t* router_q8 = nullptr; const __half *router_qs = nullptr, *router_qb = nullptr;   // [E][H] bytes, [E][H/64] scales / biases
    const uint8_t* sg_q8 = nullptr; const __half *sg_qs = nullptr, *sg_qb = nullptr;               // [H] bytes, [H/64]
    int M, H, E;
    __half* p;                           // normed rows out [M][H]
    __half* logits;                      // [M][E]
    __half* sgl;                         // [M] shared-expert gate logit
    int topk; int* inds; __half* scores; // [M][topk] routing result (written by the last CTA)
    MoeLists lists; unsigned* counter;
    unsigned* group_counter;             // [ceil(M/8)] tickets of the row groups, zero between launches
    int no_route = 0;                    // 1: stop after the logits; the consumer (fused expert kernel) routes from them itself
    EpDispatch epd;                      // expert-parallel: the last CTA sends the rows and indices to every rank instead of building lists
    int ep_rows_sent = 0;                // expert-parallel, many-row router: the norm kernel has sent the rows already; only the indices remain
    PfList pf;                           // static prefetch (every CTA)
};

// Peer pointers of the expert-parallel exchange (ep_exchange.cu): entry d is rank d's buffer as mapped into this
// process (entry `rank` is the local one).  pbuf: gathered normed rows [world*M][H]; ibuf: gathered routing indices
// [world*M][top_k]; dbuf: the pair outputs of the OWNER's rows [M*top_k][H]; flags: [0,8) dispatch, [8,16) combine.
struct EpPeers {
    __half* pbuf[8]; int* ibuf[8]; __half* dbuf[8]; unsigned* flags[8];
    unsigned* ctr;                       // local step counter (all ranks advance it in lockstep)
    int world, rank;
};

struct ExpertArgs {
    int lg_slices = 0;                   // log2(K/256), filled by the launcher
    unsigned* err = nullptr;             // set to 1 if a bounded wait on a bulk copy gave up
    Q4R gu, down;                        // expert slabs, repacked: gate/up paired tiles (I/8 per expert), down tiles (H/16 per expert)
    Q4R sh_gu, sh_down;
    MoeLists lists;
    const __half* p;                     // [M][H] normed rows
    __half* hbuf;                        // [(M*topk + M)][I]
    __half* dbuf;                        // [(M*topk + M)][H]
    int M, H, I, topk;
    const __half* rlogits = nullptr;     // fused kernel, route_here: router logits [E] of the row; every CTA routes from them itself
    int E = 0; int route_here = 0;       //   (deterministic, so all CTAs agree) instead of waiting for a routing tail in the router kernel
    int* inds_out = nullptr; __half* scores_out = nullptr;   //   CTA (0,0) publishes the result
    int lg_slices2 = 0;                  // fused kernel: log2(I/256) of the down phase
    unsigned* slot_sync = nullptr;       // fused kernel: [2][top_k + 1] counters, zero between launches
    int nstages = 1;                     // weight stages per CTA (2: a CTA walks several expert slots, filled by the launcher)
    int M_shared = -1;                   // rows the shared expert runs on (-1: all M) and where they start in p:
    int shared_row0 = 0;                 // expert-parallel calls see every rank's rows in p but own only some
    const __half* scores; const __half* sgl;   // combine inputs (down kernel)
    __half* resid;                       // residual stream updated in place, or nullptr ...
    __half* out;                         // ... then the block output goes here
    unsigned* tile_counter;              // [H/16] tickets, zero between launches; nullptr: no fused combine (dbuf only)
    // expert-parallel down projection: a routed pair's output row goes to the pair owner's buffer over peer memory
    // (rank = pair / ep_pairs_per_rank, row inside it = pair % ep_pairs_per_rank); nullptr entries: everything local
    __half* peer_dbuf[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int ep_pairs_per_rank = 0;
    EpSignal ep_sig;                     // down kernel: its last CTA raises the combine flags
    PfList pf;                           // static prefetch (gate/up kernel: next layer's in-projection)
    // many-row kernels: the normed rows in paired order + their group sums (gate/up input), and the chunk sums of the
    // SwiGLU rows ([(M*topk + M)][I/8], written by gate/up, read by down; hbuf is then in paired order too)
    const __half* xq = nullptr; const float* sxq = nullptr; float* csum = nullptr;
};

struct GdnArgs {
    const __half* inproj; int ld;        // [M][ld]: qkv | z | b | a
    const float* conv_w; const float* A_log; const float* dt_bias;
    int Hk, Hv; float eps;
    StreamTable tab; int gdn_index;      // which GDN layer (index among GDN layers)
    const SegDesc* segs;
    __half* y;                           // [M][Hv*128]
    // two-kernel form for segments of many rows: row -> segment, and the scratch between the kernels
    const int* row_seg = nullptr;
    __half* qk = nullptr;                // [M][2*Hk*128] normed, scaled q | k
    __half* vc = nullptr;                // [M][Hv*128] conv + SiLU of v
    float2* gb = nullptr;                // [M][Hv] (decay, beta)
};

struct AttnArgs {
    const __half* inproj; int ld;        // [M][ld]: q(+gate) | k | v
    const __half* q_norm; const __half* k_norm;
    int NH, KV; float eps, theta;
    StreamTable tab; int attn_index;     // index among attention layers
    int n_attn_layers, page_size;
    __half* kv_pool;
    const SegDesc* segs; const int* row_seg; const int* row_off;   // per row: segment, offset inside it
    const int* row_pos_override;         // optional explicit positions (operator tests) or nullptr
    __half* qrot;                        // [M][NH][256]
    float* part_o; float* part_ml;       // split partials
    int nsplit;
    __half* gated;                       // [M][NH*256]
    int M;
};

#ifdef __CUDACC__
// position of row m; address of (stream slot, position, K=0 / V=1, kv head) in the paged arena
__device__ __forceinline__ int row_position(const AttnArgs& a, int m) {
    if (a.row_pos_override) return a.row_pos_override[m];
    const SegDesc seg = a.segs[a.row_seg[m]];
    return a.tab.kv_len[seg.slot] + a.row_off[m];
}
__device__ __forceinline__ __half* kv_ptr(const AttnArgs& a, int slot, int pos, int which, int kvh) {
    int page = a.tab.page_table[(size_t)slot * a.tab.max_pages + pos / a.page_size];
    size_t page_elems = (size_t)a.n_attn_layers * 2 * a.KV * a.page_size * ATT_D;
    return a.kv_pool + (size_t)page * page_elems +
           ((((size_t)a.attn_index * 2 + which) * a.KV + kvh) * a.page_size + (pos % a.page_size)) * ATT_D;
}
#endif

struct StepEndArgs {
    StreamTable tab; const SegDesc* segs; int nsegs;
    const int* out_tok; int* tok_in; int* hist; int* hist_pos; int hist_cap; int M;
};

int sm_count();
// ---- the one-kernel decode step (step_persistent.cu) ----
struct PsGeom {
    int G;                                  // CTAs (one per multiprocessor)
    int H, I, E, topk, V;
    int Hk, Hv, NH, KV;
    int keyDim, valDim, convDim, gdn_in, attn_in, attn_out;
    int S_h, S_i;                           // 256-wide slices of K = H, K = I
    int gu_spp;                             // CTAs per expert slot in the gate/up phase
    int rows_per_sm;                        // gdn state rows per CTA (multiple of 4)
    int router_spr;                         // ring slots per router row
};
struct PLayer {                             // one layer's weights as the step kernel reads them (an array of these lives on the device)
    int is_attn, type_index;
    const __half *in_norm, *post_norm;
    Q4R r_in, r_out;
    const float *conv_w, *A_log, *dt_bias; const __half* gdn_norm; const float* gdn_norm32;
    const __half *q_norm, *k_norm;
    const __half *router, *shared_gate;     // fp16 forms only
    Q4R r_gu, r_down, r_sh_gu, r_sh_down;
};
struct PStepArgs {
    PsGeom geom;
    const PLayer* layers; int n_layers;
    const __half* embed; const __half* final_norm; Q4R lm_head;
    float eps, theta;
    StreamTable tab; const SegDesc* segs;
    __half* kv_pool; int n_attn_layers, page_size, nsplit;
    int *tok_in, *out_tok, *hist, *hist_pos; int hist_cap;
    unsigned* step_seq;                     // sequence number of the next step (device word, >= 1)
    // exchange lines (16 B each): per layer a block of x_stride lines, plus one block after the last layer
    int x_reps; size_t x_rep_stride;        // every exchange line exists in x_reps copies, x_rep_stride lines apart
    uint4* xbuf; size_t x_stride; int x_off_h, x_off_in, x_off_mix, x_off_hm, x_off_lg, x_off_hb, x_off_arg;
    uint4* xatt; size_t xatt_stride;        // attention partials, one block per attention layer
    unsigned* err; unsigned* abort_flag;
    uint32_t* timeline;                     // profiling: [CTA][layer + 1][24] nanosecond stamps, or nullptr
};
bool ps_plan(PsGeom& g, int n_sm);           // fills the derived fields; false if the step kernel cannot run this geometry here
int launch_step_persistent(const PStepArgs& a, cudaStream_t st);   // cooperative launch; returns a cudaError_t

void launch_dense(int pro, int epi, const DenseArgs& a, cudaStream_t st, bool pdl);
// many-row forms (more than 8 rows per call); the bool launchers return false when the shape is not covered
bool launch_dense_rows(int pro, int epi, const DenseArgs& a, cudaStream_t st);
void launch_rows_prep_plain(const __half* x, int ldx, int M, int K, __half* xq, float* sxq, cudaStream_t st);
// prefill mode: the experts of a prompt chunk as grouped GEMMs on the tensor cores (pair lists as built by the router); hbuf in natural order
bool launch_expert_tc_gateup(const ExpertArgs& a, cudaStream_t st);
bool launch_expert_tc_down(const ExpertArgs& a, cudaStream_t st);
// router for many rows: a.h holds rows that are already normed; logits kernel + routing / pair lists kernel
bool launch_router_rows(const RouterArgs& a, cudaStream_t st);
bool launch_router_mma(const RouterArgs& a, cudaStream_t st);    // prefill mode, fp16 router: logits on the tensor cores
bool launch_expert_rows_gateup(const ExpertArgs& a, cudaStream_t st);
bool launch_expert_rows_down(const ExpertArgs& a, cudaStream_t st);
void launch_moe_combine(const __half* dbuf, const __half* shared_rows, const __half* scores, const __half* sgl, int M, int H, int topk,
                        __half* resid, __half* out, cudaStream_t st);
// many-row GEMM on tcgen05 tensor cores with the accumulator in tensor memory (N % 16 == 0, K % 256 == 0); 0 or an error code
int launch_gemm_tc(const Q4R& q, int N, int K, int M, const __half* x, int ldx, __half* y, int ldy, bool add_to_y, unsigned* err, cudaStream_t st);
// speculative-sampling rows on fp16 logits [M][V]: categorical draw, draw without the draft token, accept flag
void launch_sample_rows(const __half* logits, const float* adj /*[V] added to every row, or nullptr*/, const int* draft, int* samp_full, int* samp_resid, int* accept, int M, int V,
                        float invT, float top_p, uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, cudaStream_t st);
// lm_head + argmax whose scratch is a fixed module-scope device array; returns 0 or a cudaError_t
int launch_head_static(const DenseArgs& a, cudaStream_t st);
int head_static_max_rows();
void launch_embed(const __half* embed, const int* tokens, int M, int H, int vocab, __half* h, cudaStream_t st);
void launch_embed_dequant_q4(const uint32_t* w, const __half* s, const __half* b, __half* out, int64_t vocab, int H, cudaStream_t st);
void launch_router(const RouterArgs& a, cudaStream_t st, bool pdl);
void launch_expert_gateup(const ExpertArgs& a, int nslots, cudaStream_t st, bool pdl);
void launch_expert_down(const ExpertArgs& a, int nslots, cudaStream_t st, bool pdl);
// batch-1 decode: gate/up and down in ONE launch (a per-slot barrier between the phases); false if the shapes do not fit it
bool launch_expert_fused(const ExpertArgs& a, cudaStream_t st, bool pdl);
bool expert_fused_applicable(const ExpertArgs& a);      // the shape test launch_expert_fused applies
// expert-parallel exchange (ep_exchange.cu)
void launch_ep_lists(const EpPeers& P, int npairs, int e0, int e1, const MoeLists& lists, int layer, unsigned* err, cudaStream_t st);
void launch_ep_combine(const EpPeers& P, const __half* shared_rows, const __half* scores, const __half* sgl, int M, int H, int topk,
                       __half* resid, __half* out, int layer, unsigned* err, cudaStream_t st);
void launch_ep_step_end(unsigned* ctr, cudaStream_t st);
void launch_gdn_core(const GdnArgs& a, int nsegs, cudaStream_t st, bool pdl);
// prefill-mode attention of one stream's chunk on the tensor cores (after launch_attn_prep); false: call not covered
bool launch_attn_prefill(const AttnArgs& a, int nsegs, cudaStream_t st);
void launch_gdn_rows(const GdnArgs& a, int M, int nsegs, cudaStream_t st);   // the same result by k_gdn_prep + k_gdn_scan (needs the scratch fields)
void launch_attn_prep(const AttnArgs& a, cudaStream_t st);
// q/k prep (when every row is its stream's only row) + split-KV decode + merge in one launch; counters: M*KV zeros
void launch_attn_fused(const AttnArgs& a, bool prep, unsigned* counters, cudaStream_t st, bool pdl);
void launch_step_end(const StepEndArgs& a, cudaStream_t st);
// xq / sxq (optional): the normed rows also in the prepared form of the many-row kernels
void launch_final_norm(const __half* h, const __half* w, float eps, int M, int H, __half* out, cudaStream_t st, __half* xq = nullptr, float* sxq = nullptr);
// expert-parallel: the normed rows also go into every rank's gather buffer (RouterArgs::ep_rows_sent then tells the routing kernel)
void launch_final_norm_ep(const __half* h, const __half* w, float eps, int M, int H, __half* out, const EpDispatch& epd, cudaStream_t st);
void launch_wait_probe(unsigned* err, cudaStream_t st);   // test hook: a bounded wait that runs out sets bit 2 of *err
int64_t kernel_launch_count();
void count_launch();
void count_launches(int64_t n);
// run `fn` (one kernel launch) between the profiling events of `tag` when profiling is on, and count it
void profile_launch(const char* tag, cudaStream_t st, const std::function<int()>& fn);
void profile_start();
int profile_report(char* buf, size_t cap);

// synthetic data + quantiser (synth.cu)
uint64_t tensor_seed(uint64_t base_seed, const char* name);
void launch_synth_f16(uint64_t tseed, int64_t n, float mean, float std, __half* out, cudaStream_t st);
void launch_synth_f32(uint64_t tseed, int64_t n, float mean, float std, float* out, cudaStream_t st);
void launch_synth_q4(uint64_t tseed, int64_t N, int64_t K, float std, uint32_t* packed, __half* s, __half* b, cudaStream_t st);
void launch_quantize_q4(const __half* w, int64_t N, int64_t K, uint32_t* packed, __half* s, __half* b, cudaStream_t st);
void host_synth_tokens(uint64_t tseed, int64_t n, int32_t vocab, int32_t* out);
// MLX affine layout -> fragment-major layout; pair != 0: tile = 8 rows of A + the same 8 rows of B
void launch_repack_q4(const Q4W& a, const Q4W* b_pair, uint4* wr, uint4* sr, cudaStream_t st);

}  // namespace sl
