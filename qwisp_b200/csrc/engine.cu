// engine.cu -- engine / stream objects and the C ABI of libseedless_b200.so.
//
// Host-side orchestration of one step (the op order of the reference's fused step,
// swift/Sources/QwispCore/SeedlessFusedVerify.swift:3455-3549 and :3832-3912):
//   embed -> per layer [ rmsnorm -> mixer (GDN | attention) -> +resid -> rmsnorm -> MoE -> +resid ]
//         -> rmsnorm -> lm_head -> argmax
// All state stays on the device; a decode step reads back only int32 token ids.
#include "../../include/seedless_b200.h"
#include "gemv.cuh"
#include "kernels.h"
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

using namespace sl;

namespace {

constexpr int NSPLIT = 64;          // KV splits of the decode attention

struct Tensor { void* ptr; size_t bytes; };

struct LayerW {
    bool is_attn = false;
    int type_index = 0;             // index among layers of the same kind
    const __half *in_norm = nullptr, *post_norm = nullptr;
    Q4W in_proj;                    // GDN: qkv|z|b|a rows; attention: q|k|v rows
    const float *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr;
    const __half* gdn_norm = nullptr;
    const float* gdn_norm32 = nullptr;   // set when the checkpoint stores this weight as f32: the gated norm then runs in f32
    Q4W out_proj;                   // GDN out_proj / attention o_proj
    const __half *q_norm = nullptr, *k_norm = nullptr;
    const __half *router = nullptr, *shared_gate = nullptr;
    // 8-bit group-64 router / shared gate (the checkpoint's layout); when set they are used instead of the fp16 pair
    const uint8_t *router_q8 = nullptr, *sg_q8 = nullptr;
    const __half *router_qs = nullptr, *router_qb = nullptr, *sg_qs = nullptr, *sg_qb = nullptr;
    Q4W gate, up, down, sh_gate, sh_up, sh_down;
    // fragment-major copies the kernels read (gate/up fused into paired tiles)
    Q4R r_in, r_out, r_gu, r_down, r_sh_gu, r_sh_down;
};

}  // namespace

struct sl_engine {
    sl_config cfg{};
    int H = 0, E = 0, I = 0, topk = 0, V = 0;
    int keyDim = 0, valDim = 0, convDim = 0, gdn_in = 0, attn_in = 0, attn_out = 0;
    int n_gdn = 0, n_attn = 0;
    bool hybrid = false;            // set for the duration of a prefill-mode call: dense projections on the tensor-core GEMM
    cudaStream_t own_stream = nullptr, stream = nullptr;
    std::map<std::string, Tensor> tensors;
    std::vector<void*> allocs;
    std::vector<LayerW> layers;
    const __half *embed = nullptr, *final_norm = nullptr;
    Q4W lm_head; Q4R r_lm_head;
    // scratch (sized by max_rows)
    __half *h = nullptr, *p = nullptr, *inproj = nullptr, *mix = nullptr, *rlogits = nullptr, *sgl = nullptr, *scores = nullptr;
    __half *hbuf = nullptr, *dbuf = nullptr, *normed = nullptr, *qrot = nullptr, *opx = nullptr, *opy = nullptr;
    // many-row kernels: prepared rows of a dense projection / of the experts' input, their group sums, chunk sums of the SwiGLU rows
    __half *xq = nullptr, *xq_p = nullptr; float *sxq = nullptr, *sx_p = nullptr, *csum = nullptr;
    __half *gdn_qk = nullptr, *gdn_vc = nullptr; float2* gdn_gb = nullptr;    // between k_gdn_prep and k_gdn_scan
    __half* logits = nullptr; int logits_rows = 0;
    int* inds = nullptr; MoeLists lists{};
    float *part_o = nullptr, *part_ml = nullptr, *pval = nullptr;
    int *pidx = nullptr, *out_tok = nullptr, *tok_in = nullptr, *hist = nullptr, *hist_pos = nullptr;
    int *row_seg = nullptr, *row_off = nullptr, *row_pos = nullptr;
    unsigned* counters = nullptr; unsigned* tile_counters = nullptr; unsigned* att_counters = nullptr; unsigned* err_flag = nullptr; unsigned* err_host = nullptr; float* adj_buf = nullptr; int* samp_buf = nullptr; unsigned* slot_sync = nullptr; unsigned* router_groups = nullptr;
    bool use_route_in_experts = true;   // with the fused kernel: routing done by its CTAs (SL_FLAG_ROUTE_IN_ROUTER: by the router's last CTA)
    bool use_rows = true;           // calls with more than 8 rows use the many-row kernels (SL_FLAG_PASS_KERNELS turns it off)
    bool use_fused_experts = true;  // batch-1 decode: gate/up + down in one launch (SL_FLAG_SPLIT_EXPERTS turns it off)
    // expert-parallel decode (experts [ep_e0, ep_e1) are this rank's; see sl_ep_init)
    int ep_rank = 0, ep_world = 1, ep_rows = 0, ep_e0 = 0, ep_e1 = 0;
    bool ep_step = false;
    void* ep_comm = nullptr;
    EpPeers ep_peers{};               // peer-memory exchange buffers (own + mapped peers'), see ep_exchange.cu
    void* ep_region = nullptr;        // this rank's exchange region (shared with the peers through CUDA IPC)
    void* ep_mapped[8] = {};          // peers' regions as mapped here
    int ep_layer_seq = 0;             // MoE layers enqueued so far in the step being built
    SegDesc* segs = nullptr;
    int hist_cap = 0;
    // pinned staging
    int* pin_i = nullptr; size_t pin_ints = 0;
    // streams
    StreamTable tab{};
    __half* kv_pool = nullptr;
    std::vector<int> free_pages;
    std::vector<int> free_slots;
    // decode graphs keyed by rows (each segment one row)
    std::map<int, cudaGraphExec_t> graphs;
    std::map<int, int> graph_kernels;   // kernels inside each captured step (so replays are counted too)
    std::map<int, int> eager_runs;
    bool use_graph = true;
    bool use_prefetch = false;      // L2 prefetch of the weights later kernels read (SL_FLAG_L2_PREFETCH); slower now that
                                    // every kernel starts its own weight copies ahead of the launch wait
    bool use_pdl = true;            // programmatic dependent launch between the kernels of a step (SL_FLAG_NO_PDL turns it off)
    // the one-kernel decode step (step_persistent.cu): used for single-stream decode steps when the geometry fits
    // Off by default: measured on B200 it is the slower of the two assemblies (its six all-to-all activation exchanges
    // per layer cost more than the kernel boundaries they replace); SL_FLAG_STEP_KERNEL / sl_engine_use_persistent(e, 1) selects it
    bool ps_ok = false, use_persistent = false;
    PStepArgs ps{};
    uint32_t* ps_timeline = nullptr;
    bool poisoned = false, inject = false;
    std::string fault;
};

struct sl_stream {
    sl_engine* e;
    int slot;
    int max_seq_len;
    int kv_len;
    int parity;
    std::vector<int> pages;
    int calls = 0;                  // forward / step calls (chained steps count one each) since creation: what a snapshot remembers
};

struct sl_fullsnap {
    int kv_len;
    float* state;      // [n_gdn][Hv*128*128]
    __half* hist;      // [n_gdn][3*convDim]
};

namespace {

int32_t poison(sl_engine* e, const char* what, cudaError_t err) {
    if (!e->poisoned) {
        e->poisoned = true;
        e->fault = std::string(what) + ": " + cudaGetErrorString(err);
    }
    return SL_ERR_CUDA;
}
int32_t poison_msg(sl_engine* e, const std::string& what) {
    if (!e->poisoned) { e->poisoned = true; e->fault = what; }
    return SL_ERR_CUDA;
}
#define CU(e, call)                                         \
    do {                                                    \
        cudaError_t _err = (call);                          \
        if (_err != cudaSuccess) return poison((e), #call, _err); \
    } while (0)

int32_t guard(sl_engine* e) {
    if (!e) return SL_ERR_INVALID;
    if (e->poisoned) return SL_ERR_POISONED;
    if (e->inject) {
        e->poisoned = true;
        e->fault = "injected failure (test hook)";
        e->inject = false;
        return SL_ERR_CUDA;
    }
    return SL_OK;
}

bool device_ok() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return false; }
    return true;
}

template <typename T>
int32_t dalloc(sl_engine* e, T** out, size_t count) {
    void* p = nullptr;
    size_t bytes = count * sizeof(T);
    if (bytes == 0) bytes = 16;
    CU(e, cudaMalloc(&p, bytes));
    e->allocs.push_back(p);
    *out = reinterpret_cast<T*>(p);
    return SL_OK;
}

int32_t reg_tensor(sl_engine* e, const std::string& name, void* ptr, size_t bytes) {
    e->tensors[name] = Tensor{ptr, bytes};
    return SL_OK;
}

// one q4 tensor with rows possibly shared by several named sub-tensors (row ranges)
int32_t alloc_q4(sl_engine* e, Q4W& q, int64_t N, int K, const std::vector<std::pair<std::string, int64_t>>& parts) {
    uint32_t* w; __half *s, *b;
    int32_t rc;
    if ((rc = dalloc(e, &w, (size_t)N * K / 8))) return rc;
    if ((rc = dalloc(e, &s, (size_t)N * K / 64))) return rc;
    if ((rc = dalloc(e, &b, (size_t)N * K / 64))) return rc;
    q.w = w; q.s = s; q.b = b; q.N = N; q.K = K;
    int64_t row = 0;
    for (auto& pr : parts) {
        reg_tensor(e, pr.first + ".w", w + row * (K / 8), (size_t)pr.second * K / 8 * 4);
        reg_tensor(e, pr.first + ".s", s + row * (K / 64), (size_t)pr.second * K / 64 * 2);
        reg_tensor(e, pr.first + ".b", b + row * (K / 64), (size_t)pr.second * K / 64 * 2);
        row += pr.second;
    }
    return SL_OK;
}
template <typename T>
int32_t alloc_plain(sl_engine* e, const T** out, const std::string& name, size_t count) {
    T* p; int32_t rc;
    if ((rc = dalloc(e, &p, count))) return rc;
    *out = p;
    return reg_tensor(e, name, p, count * sizeof(T));
}

// the GEMV family needs K/256 to be a power of two (a warp's slice index is taken with a mask)
static bool k_ok(int64_t K) { return K >= 256 && K <= 4096 && K % 256 == 0 && (((K >> 8) & ((K >> 8) - 1)) == 0); }

bool config_ok(const sl_config& c) {
    if (!k_ok(c.hidden) || !k_ok(c.moe_inter) || !k_ok((int64_t)c.gdn_v_heads * GDN_DV) || !k_ok((int64_t)c.attn_heads * ATT_D)) return false;
    if (c.hidden <= 0 || c.hidden % 256 || c.hidden > 4096) return false;
    if (c.moe_inter <= 0 || c.moe_inter % 256 || c.moe_inter > 4096) return false;
    if (c.n_layers <= 0 || c.attn_every <= 0) return false;
    if (c.vocab <= 0 || c.vocab % 16) return false;
    if (c.n_experts <= 0 || c.n_experts > 256 || c.n_experts % 8) return false;
    if (c.top_k <= 0 || c.top_k > c.n_experts || c.top_k > 16) return false;
    if (c.gdn_k_heads <= 0 || c.gdn_v_heads % c.gdn_k_heads) return false;
    if ((c.gdn_v_heads * GDN_DV) % 256 || (c.gdn_v_heads * GDN_DV) > 4096) return false;
    if (c.gdn_v_heads % 16) return false;           // b / a rows form whole 16-row tiles
    if (c.attn_kv_heads <= 0 || c.attn_heads != 8 * c.attn_kv_heads) return false;
    if ((c.attn_heads * ATT_D) > 4096) return false;
    if (c.max_rows <= 0 || c.max_rows > 1024) return false;
    if (c.max_streams <= 0 || c.max_streams > 1024) return false;
    if (c.kv_page_size <= 0 || c.kv_page_size % 32) return false;
    if (c.kv_pages <= 0) return false;
    return true;
}

int32_t build_layout(sl_engine* e) {
    const sl_config& c = e->cfg;
    e->H = c.hidden; e->E = c.n_experts; e->I = c.moe_inter; e->topk = c.top_k; e->V = c.vocab;
    e->keyDim = c.gdn_k_heads * GDN_DK; e->valDim = c.gdn_v_heads * GDN_DV; e->convDim = 2 * e->keyDim + e->valDim;
    e->gdn_in = e->convDim + e->valDim + 2 * c.gdn_v_heads;
    e->attn_in = c.attn_heads * 2 * ATT_D + 2 * c.attn_kv_heads * ATT_D;
    e->attn_out = c.attn_heads * ATT_D;
    const int H = e->H, E = e->E, I = e->I;
    int32_t rc;
    if ((rc = alloc_plain(e, &e->embed, "embed", (size_t)c.vocab * H))) return rc;
    if ((rc = alloc_plain(e, &e->final_norm, "final_norm", (size_t)H))) return rc;
    if ((rc = alloc_q4(e, e->lm_head, c.vocab, H, {{"lm_head", c.vocab}}))) return rc;
    e->layers.resize(c.n_layers);
    for (int i = 0; i < c.n_layers; ++i) {
        LayerW& L = e->layers[i];
        std::string p = "L" + std::to_string(i) + ".";
        L.is_attn = ((i + 1) % c.attn_every) == 0;
        L.type_index = L.is_attn ? e->n_attn++ : e->n_gdn++;
        if ((rc = alloc_plain(e, &L.in_norm, p + "in_norm", (size_t)H))) return rc;
        if ((rc = alloc_plain(e, &L.post_norm, p + "post_norm", (size_t)H))) return rc;
        if (!L.is_attn) {
            if ((rc = alloc_q4(e, L.in_proj, e->gdn_in, H,
                               {{p + "gdn.in_proj_qkv", e->convDim}, {p + "gdn.in_proj_z", e->valDim},
                                {p + "gdn.in_proj_b", c.gdn_v_heads}, {p + "gdn.in_proj_a", c.gdn_v_heads}}))) return rc;
            if ((rc = alloc_plain(e, &L.conv_w, p + "gdn.conv_w", (size_t)e->convDim * CONV_K))) return rc;
            if ((rc = alloc_plain(e, &L.A_log, p + "gdn.A_log", (size_t)c.gdn_v_heads))) return rc;
            if ((rc = alloc_plain(e, &L.dt_bias, p + "gdn.dt_bias", (size_t)c.gdn_v_heads))) return rc;
            if ((rc = alloc_plain(e, &L.gdn_norm, p + "gdn.norm", (size_t)GDN_DV))) return rc;
            if ((rc = alloc_q4(e, L.out_proj, H, e->valDim, {{p + "gdn.out_proj", H}}))) return rc;
        } else {
            if ((rc = alloc_q4(e, L.in_proj, e->attn_in, H,
                               {{p + "attn.q_proj", c.attn_heads * 2 * ATT_D}, {p + "attn.k_proj", c.attn_kv_heads * ATT_D},
                                {p + "attn.v_proj", c.attn_kv_heads * ATT_D}}))) return rc;
            if ((rc = alloc_q4(e, L.out_proj, H, e->attn_out, {{p + "attn.o_proj", H}}))) return rc;
            if ((rc = alloc_plain(e, &L.q_norm, p + "attn.q_norm", (size_t)ATT_D))) return rc;
            if ((rc = alloc_plain(e, &L.k_norm, p + "attn.k_norm", (size_t)ATT_D))) return rc;
        }
        if ((rc = alloc_plain(e, &L.router, p + "moe.router", (size_t)E * H))) return rc;
        if ((rc = alloc_plain(e, &L.shared_gate, p + "moe.shared_gate", (size_t)H))) return rc;
        if ((rc = alloc_q4(e, L.gate, (int64_t)E * I, H, {{p + "moe.gate_proj", (int64_t)E * I}}))) return rc;
        if ((rc = alloc_q4(e, L.up, (int64_t)E * I, H, {{p + "moe.up_proj", (int64_t)E * I}}))) return rc;
        if ((rc = alloc_q4(e, L.down, (int64_t)E * H, I, {{p + "moe.down_proj", (int64_t)E * H}}))) return rc;
        if ((rc = alloc_q4(e, L.sh_gate, I, H, {{p + "moe.shared_gate_proj", I}}))) return rc;
        if ((rc = alloc_q4(e, L.sh_up, I, H, {{p + "moe.shared_up_proj", I}}))) return rc;
        if ((rc = alloc_q4(e, L.sh_down, H, I, {{p + "moe.shared_down_proj", H}}))) return rc;
    }
    return SL_OK;
}

int32_t build_runtime(sl_engine* e) {
    const sl_config& c = e->cfg;
    const int R = c.max_rows, H = e->H;
    int32_t rc;
    CU(e, cudaStreamCreateWithFlags(&e->own_stream, cudaStreamNonBlocking));
    e->stream = e->own_stream;
    size_t in_w = (size_t)(e->gdn_in > e->attn_in ? e->gdn_in : e->attn_in);
    size_t mix_w = (size_t)(e->valDim > e->attn_out ? e->valDim : e->attn_out);
    size_t prow = (size_t)R * e->topk + R;
    if ((rc = dalloc(e, &e->h, (size_t)R * H))) return rc;
    if ((rc = dalloc(e, &e->p, (size_t)R * H))) return rc;
    if ((rc = dalloc(e, &e->normed, (size_t)R * (e->valDim > H ? e->valDim : H)))) return rc;   // also the gated-norm rows of prefill mode
    {
        const size_t wmax = (size_t)(mix_w > (size_t)H ? mix_w : (size_t)H);
        if ((rc = dalloc(e, &e->xq, (size_t)R * wmax))) return rc;
        if ((rc = dalloc(e, &e->sxq, (size_t)R * (wmax / 64)))) return rc;
        if ((rc = dalloc(e, &e->xq_p, (size_t)R * H))) return rc;
        if ((rc = dalloc(e, &e->sx_p, (size_t)R * (H / 64)))) return rc;
        if ((rc = dalloc(e, &e->csum, prow * (size_t)(e->I / 8)))) return rc;
        if ((rc = dalloc(e, &e->gdn_qk, (size_t)R * 2 * e->keyDim))) return rc;
        if ((rc = dalloc(e, &e->gdn_vc, (size_t)R * e->valDim))) return rc;
        if ((rc = dalloc(e, &e->gdn_gb, (size_t)R * c.gdn_v_heads))) return rc;
    }
    if ((rc = dalloc(e, &e->opx, (size_t)R * H))) return rc;
    if ((rc = dalloc(e, &e->opy, (size_t)R * H))) return rc;
    if ((rc = dalloc(e, &e->inproj, (size_t)R * in_w))) return rc;
    if ((rc = dalloc(e, &e->mix, (size_t)R * mix_w))) return rc;
    if ((rc = dalloc(e, &e->rlogits, (size_t)R * e->E))) return rc;
    if ((rc = dalloc(e, &e->sgl, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->scores, (size_t)R * e->topk))) return rc;
    if ((rc = dalloc(e, &e->inds, (size_t)R * e->topk))) return rc;
    if ((rc = dalloc(e, &e->hbuf, prow * e->I))) return rc;
    if ((rc = dalloc(e, &e->dbuf, prow * H))) return rc;
    if ((rc = dalloc(e, &e->qrot, (size_t)R * c.attn_heads * ATT_D))) return rc;
    if ((rc = dalloc(e, &e->part_o, (size_t)R * c.attn_heads * NSPLIT * ATT_D))) return rc;
    if ((rc = dalloc(e, &e->part_ml, (size_t)R * c.attn_heads * NSPLIT * 2))) return rc;
    if ((rc = dalloc(e, &e->pval, (size_t)R * (e->V / 16)))) return rc;
    if ((rc = dalloc(e, &e->pidx, (size_t)R * (e->V / 16)))) return rc;
    if ((rc = dalloc(e, &e->out_tok, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->tok_in, (size_t)R))) return rc;
    e->hist_cap = 1 << 16;
    if ((rc = dalloc(e, &e->hist, (size_t)e->hist_cap))) return rc;
    if ((rc = dalloc(e, &e->hist_pos, (size_t)1))) return rc;
    if ((rc = dalloc(e, &e->row_seg, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->row_off, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->row_pos, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->counters, (size_t)8))) return rc;
    if ((rc = dalloc(e, &e->segs, (size_t)R))) return rc;
    if ((rc = dalloc(e, &e->lists.n_active, (size_t)1))) return rc;
    if ((rc = dalloc(e, &e->lists.slot_expert, (size_t)256))) return rc;
    if ((rc = dalloc(e, &e->lists.slot_off, (size_t)256))) return rc;
    if ((rc = dalloc(e, &e->lists.slot_cnt, (size_t)256))) return rc;
    if ((rc = dalloc(e, &e->lists.pairs, (size_t)R * e->topk))) return rc;
    if ((rc = dalloc(e, &e->tile_counters, (size_t)(H / 16)))) return rc;
    CU(e, cudaMemset(e->tile_counters, 0, (size_t)(H / 16) * sizeof(unsigned)));
    CU(e, cudaMemset(e->counters, 0, 8 * sizeof(unsigned)));
    if ((rc = dalloc(e, &e->samp_buf, (size_t)4 * R))) return rc;
    if ((rc = dalloc(e, &e->router_groups, (size_t)(R / 8 + 2)))) return rc;
    CU(e, cudaMemset(e->router_groups, 0, (size_t)(R / 8 + 2) * sizeof(unsigned)));
    if ((rc = dalloc(e, &e->slot_sync, (size_t)64))) return rc;
    CU(e, cudaMemset(e->slot_sync, 0, 64 * sizeof(unsigned)));
    // Kernels whose bounded wait runs out leave a code here.  The word lives in mapped page-locked host
    // memory, so it costs nothing while all is well and the host sees it after the synchronisation that
    // ends every call, without a copy.
    CU(e, cudaHostAlloc((void**)&e->err_host, 4 * sizeof(unsigned), cudaHostAllocMapped));
    memset(e->err_host, 0, 4 * sizeof(unsigned));
    CU(e, cudaHostGetDevicePointer((void**)&e->err_flag, e->err_host, 0));
    if ((rc = dalloc(e, &e->att_counters, (size_t)R * c.attn_kv_heads))) return rc;
    CU(e, cudaMemset(e->att_counters, 0, (size_t)R * c.attn_kv_heads * sizeof(unsigned)));
    CU(e, cudaMemset(e->hist_pos, 0, sizeof(int)));
    e->pin_ints = (size_t)R * 8 + 64;
    CU(e, cudaMallocHost(&e->pin_i, e->pin_ints * sizeof(int)));
    // stream tables
    const int S = c.max_streams;
    StreamTable& t = e->tab;
    t.max_pages = c.kv_pages;
    if ((rc = dalloc(e, &t.kv_len, (size_t)S))) return rc;
    if ((rc = dalloc(e, &t.parity, (size_t)S))) return rc;
    if ((rc = dalloc(e, &t.page_table, (size_t)S * t.max_pages))) return rc;
    CU(e, cudaMemset(t.kv_len, 0, S * sizeof(int)));
    CU(e, cudaMemset(t.parity, 0, S * sizeof(int)));
    CU(e, cudaMemset(t.page_table, 0, (size_t)S * t.max_pages * sizeof(int)));
    t.state_stride_layer = (size_t)c.gdn_v_heads * GDN_DV * GDN_DK;
    t.state_stride_side = t.state_stride_layer * (e->n_gdn > 0 ? e->n_gdn : 1);
    t.state_stride_stream = 2 * t.state_stride_side;
    t.hist_stride_layer = (size_t)(CONV_K - 1) * e->convDim;
    t.hist_stride_side = t.hist_stride_layer * (e->n_gdn > 0 ? e->n_gdn : 1);
    t.hist_stride_stream = 2 * t.hist_stride_side;
    if ((rc = dalloc(e, &t.gdn_state, (size_t)S * t.state_stride_stream))) return rc;
    if ((rc = dalloc(e, &t.conv_hist, (size_t)S * t.hist_stride_stream))) return rc;
    size_t page_elems = (size_t)(e->n_attn > 0 ? e->n_attn : 1) * 2 * c.attn_kv_heads * c.kv_page_size * ATT_D;
    if ((rc = dalloc(e, &e->kv_pool, (size_t)c.kv_pages * page_elems))) return rc;
    for (int i = c.kv_pages - 1; i >= 0; --i) e->free_pages.push_back(i);
    for (int i = S - 1; i >= 0; --i) e->free_slots.push_back(i);
    // assembly switches come with the configuration (sl_config.flags), not from the environment
    e->use_route_in_experts = !(c.flags & SL_FLAG_ROUTE_IN_ROUTER);
    e->use_fused_experts = !(c.flags & SL_FLAG_SPLIT_EXPERTS);
    e->use_rows = !(c.flags & SL_FLAG_PASS_KERNELS);
    e->use_prefetch = (c.flags & SL_FLAG_L2_PREFETCH) != 0;
    e->use_pdl = !(c.flags & SL_FLAG_NO_PDL);
    e->use_graph = !(c.flags & SL_FLAG_NO_GRAPH);
    return SL_OK;
}

// allocate and fill the fragment-major copy of a (pair of) 4-bit tensor(s)
int32_t repack(sl_engine* e, const Q4W& a, const Q4W* pair, Q4R& out) {
    int64_t tiles = pair ? a.N / 8 : a.N / 16;
    uint4 *wr, *sr; int32_t rc;
    if ((rc = dalloc(e, &wr, (size_t)tiles * q4r_w_uint4(a.K)))) return rc;
    if ((rc = dalloc(e, &sr, (size_t)tiles * q4r_s_uint4(a.K)))) return rc;
    launch_repack_q4(a, pair, wr, sr, e->stream);
    out.wr = wr; out.sr = sr; out.tiles = (int)tiles; out.K = a.K;
    return SL_OK;
}
int32_t repack_all(sl_engine* e) {
    int32_t rc;
    if ((rc = repack(e, e->lm_head, nullptr, e->r_lm_head))) return rc;
    for (LayerW& L : e->layers) {
        if ((rc = repack(e, L.in_proj, nullptr, L.r_in))) return rc;
        if ((rc = repack(e, L.out_proj, nullptr, L.r_out))) return rc;
        if ((rc = repack(e, L.gate, &L.up, L.r_gu))) return rc;
        if ((rc = repack(e, L.down, nullptr, L.r_down))) return rc;
        if ((rc = repack(e, L.sh_gate, &L.sh_up, L.r_sh_gu))) return rc;
        if ((rc = repack(e, L.sh_down, nullptr, L.r_sh_down))) return rc;
    }
    CU(e, cudaStreamSynchronize(e->stream));
    CU(e, cudaGetLastError());
    return SL_OK;
}

// Set up the one-kernel decode step: the layer table on the device, the exchange lines, the sequence word.
// Leaves ps_ok false (the kernel-per-phase assembly then serves every call) when the geometry or the device does
// not fit: 8-bit router weights, too few multiprocessors for a phase, no cooperative launch.
int32_t setup_persistent(sl_engine* e) {
    const sl_config& c = e->cfg;
    for (const LayerW& L : e->layers) if (L.router_q8) return SL_OK;
    PsGeom g{};
    g.H = e->H; g.I = e->I; g.E = e->E; g.topk = e->topk; g.V = e->V;
    g.Hk = c.gdn_k_heads; g.Hv = c.gdn_v_heads; g.NH = c.attn_heads; g.KV = c.attn_kv_heads;
    g.keyDim = e->keyDim; g.valDim = e->valDim; g.convDim = e->convDim; g.gdn_in = e->gdn_in; g.attn_in = e->attn_in; g.attn_out = e->attn_out;
    if (!ps_plan(g, sm_count())) return SL_OK;
    std::vector<PLayer> host(e->layers.size());
    for (size_t i = 0; i < e->layers.size(); ++i) {
        const LayerW& L = e->layers[i]; PLayer& P = host[i];
        P.is_attn = L.is_attn ? 1 : 0; P.type_index = L.type_index;
        P.in_norm = L.in_norm; P.post_norm = L.post_norm; P.r_in = L.r_in; P.r_out = L.r_out;
        P.conv_w = L.conv_w; P.A_log = L.A_log; P.dt_bias = L.dt_bias; P.gdn_norm = L.gdn_norm; P.gdn_norm32 = L.gdn_norm32;
        P.q_norm = L.q_norm; P.k_norm = L.k_norm; P.router = L.router; P.shared_gate = L.shared_gate;
        P.r_gu = L.r_gu; P.r_down = L.r_down; P.r_sh_gu = L.r_sh_gu; P.r_sh_down = L.r_sh_down;
    }
    PLayer* dl = nullptr; int32_t rc;
    if ((rc = dalloc(e, &dl, host.size()))) return rc;
    CU(e, cudaMemcpy(dl, host.data(), host.size() * sizeof(PLayer), cudaMemcpyHostToDevice));
    PStepArgs& a = e->ps;
    a.geom = g; a.layers = dl; a.n_layers = (int)host.size();
    a.embed = e->embed; a.final_norm = e->final_norm; a.lm_head = e->r_lm_head;
    a.eps = c.rms_eps; a.theta = c.rope_theta;
    a.tab = e->tab; a.segs = e->segs; a.kv_pool = e->kv_pool; a.n_attn_layers = e->n_attn > 0 ? e->n_attn : 1; a.page_size = c.kv_page_size; a.nsplit = NSPLIT;
    a.tok_in = e->tok_in; a.out_tok = e->out_tok; a.hist = e->hist; a.hist_pos = e->hist_pos; a.hist_cap = e->hist_cap;
    // exchange lines of a layer (16 bytes carry 4 halves): residual stream in, in-projection out, mixer out,
    // residual stream after the mixer, router logits (one per half line) + shared-gate logit, SwiGLU rows; the
    // block after the last layer also holds one argmax line per CTA
    int off = 0;
    const int in_w = e->gdn_in > e->attn_in ? e->gdn_in : e->attn_in, mix_w = e->valDim > e->attn_out ? e->valDim : e->attn_out;
    a.x_off_h = off; off += e->H / 4;
    a.x_off_in = off; off += (in_w + 3) / 4;
    a.x_off_mix = off; off += mix_w / 4;
    a.x_off_hm = off; off += e->H / 4;
    a.x_off_lg = off; off += (e->E + 2) / 2;
    a.x_off_hb = off; off += (e->topk + 1) * e->I / 4;
    a.x_off_arg = off; off += g.G;
    a.x_stride = (size_t)((off + 7) & ~7);
    a.x_reps = 8;
    a.x_rep_stride = a.x_stride * (host.size() + 1);
    const size_t xlines = a.x_rep_stride * (size_t)a.x_reps;
    if ((rc = dalloc(e, &a.xbuf, xlines))) return rc;
    CU(e, cudaMemset(a.xbuf, 0, xlines * sizeof(uint4)));
    a.xatt_stride = (size_t)c.attn_heads * NSPLIT * 129;
    const size_t alines = a.xatt_stride * (size_t)(e->n_attn > 0 ? e->n_attn : 1);
    if ((rc = dalloc(e, &a.xatt, alines))) return rc;
    CU(e, cudaMemset(a.xatt, 0, alines * sizeof(uint4)));
    unsigned* words = nullptr;
    if ((rc = dalloc(e, &words, (size_t)4))) return rc;
    const unsigned init[4] = {1u, 0u, 0u, 0u};
    CU(e, cudaMemcpy(words, init, sizeof(init), cudaMemcpyHostToDevice));
    a.step_seq = words; a.abort_flag = words + 1; a.err = e->err_flag;
    e->use_persistent = (c.flags & SL_FLAG_STEP_KERNEL) != 0;
    e->ps_ok = true;
    return SL_OK;
}

// ---------------------------------------------------------------- NCCL, loaded on demand
// The library has no link-time dependency on NCCL: expert-parallel mode resolves the few entry
// points it needs from the process's libnccl.so.2 (the copy the host framework already loaded, if any).
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
    bool ok = false;
};
static NcclApi g_nccl;
static bool load_nccl() {
    if (g_nccl.ok) return true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return false;
#define SL_NCCL_SYM(field, name) *(void**)(&g_nccl.field) = dlsym(h, name); if (!g_nccl.field) return false;
    SL_NCCL_SYM(GetUniqueId, "ncclGetUniqueId") SL_NCCL_SYM(CommInitRank, "ncclCommInitRank") SL_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    SL_NCCL_SYM(AllGather, "ncclAllGather") SL_NCCL_SYM(ReduceScatter, "ncclReduceScatter")
    SL_NCCL_SYM(GroupStart, "ncclGroupStart") SL_NCCL_SYM(GroupEnd, "ncclGroupEnd") SL_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef SL_NCCL_SYM
    g_nccl.ok = true;
    return true;
}
#define NC(e, call) do { ncclResult_t _r = (call); if (_r != ncclSuccess) return poison_msg(e, std::string("NCCL: ") + g_nccl.GetErrorString(_r)); } while (0)

// ---------------------------------------------------------------- the forward pass
enum HeadMode { HEAD_NONE = 0, HEAD_NORMED = 1, HEAD_ARGMAX = 2, HEAD_LOGITS = 3 };

void pf_q4(PfList& pf, int i, const Q4R& q, size_t max_bytes = (size_t)48 << 20) {
    size_t wb = (size_t)q.tiles * q4r_w_uint4(q.K) * 16, gb = (size_t)q.tiles * q4r_s_uint4(q.K) * 16;
    if (wb > max_bytes) { wb = max_bytes; gb = 0; }
    pf.p[i] = q.wr; pf.bytes[i] = (unsigned)wb;
    if (i + 1 < 6 && gb) { pf.p[i + 1] = q.sr; pf.bytes[i + 1] = (unsigned)gb; }
}

// Router of an M-row call.  Many rows: the rows are normed once (k_final_norm), then the many-row router (logits kernel +
// routing / pair-list kernel, same bits); otherwise the one-kernel router.
// xq / sxq (optional): also leave the normed rows in the prepared form of the many-row expert kernels; returns true if it did.
bool enqueue_router(sl_engine* e, const RouterArgs& ra, int M, bool pdl, __half* xq = nullptr, float* sxq = nullptr) {
    cudaStream_t st = e->stream;
    // (expert-parallel calls take this path from 2 rows on: its routing kernel spreads the dispatch over CTAs and warps)
    // (prefill mode takes it for ANY row count: which kernels run must not depend on how a prompt is cut into calls)
    if ((M > 8 || e->hybrid || (ra.epd.sig.world > 0 && M > 1)) && e->use_rows && !ra.no_route && e->E <= 256 && ra.norm_w && ra.ldh == e->H) {
        const bool ep = ra.epd.sig.world > 0;
        if (ep) launch_final_norm_ep(ra.h, ra.norm_w, ra.eps, M, e->H, ra.p, ra.epd, st);     // the rows leave for the peers here
        else launch_final_norm(ra.h, ra.norm_w, ra.eps, M, e->H, ra.p, st, xq, sxq);
        RouterArgs rb = ra; rb.h = ra.p; rb.ldh = e->H; rb.norm_w = nullptr; rb.ep_rows_sent = ep ? 1 : 0;
        if (e->hybrid && launch_router_mma(rb, st)) return xq != nullptr;
        if (launch_router_rows(rb, st)) return xq != nullptr;
        // not covered: the one-kernel router norms the rows again from the original input
    }
    launch_router(ra, st, pdl);
    return false;
}

// Expert-parallel MoE block of a decode step.  Every rank runs the same number M of rows (its own streams);
// rank r owns experts [ep_e0, ep_e1).  Per layer (kernels of ep_exchange.cu, no collective):
//   router on the local rows, its last CTA storing the normed rows and routing indices into every rank's gather
//   buffers over peer memory -> k_ep_lists waits for all ranks' rows, groups the pairs that chose a local expert
//   -> the expert kernels run on them, the down projection storing each pair's output row straight into the pair
//   owner's buffer and raising the combine flags -> k_ep_combine waits for all ranks' outputs, combines in ascending k
//   with the shared expert (computed locally on the local rows) and the residual.
// Each pair row is computed by exactly one rank and arrives unreduced: the owner sees a single GPU's bits.
int32_t enqueue_moe_ep(sl_engine* e, const LayerW& L, RouterArgs ra, int M, __half* resid, __half* plain_out) {
    cudaStream_t st = e->stream;
    const int R = e->ep_world, r = e->ep_rank, T = R * M, topk = e->topk, H = e->H;
    const int layer = e->ep_layer_seq++;
    const EpPeers& P = e->ep_peers;
    ra.p = e->p + (size_t)r * M * H;
    ra.inds = e->inds + (size_t)r * M * topk;
    for (int d = 0; d < R; ++d) { ra.epd.pbuf[d] = P.pbuf[d]; ra.epd.ibuf[d] = P.ibuf[d]; ra.epd.sig.flags[d] = P.flags[d]; }
    ra.epd.sig.ctr = P.ctr; ra.epd.sig.world = R; ra.epd.sig.rank = r; ra.epd.sig.layer = layer;
    enqueue_router(e, ra, M, false);                   // its last CTA sends the rows and indices to every rank
    launch_ep_lists(P, T * topk, e->ep_e0, e->ep_e1, e->lists, layer, e->err_flag, st);
    ExpertArgs ea{}; ea.gu = L.r_gu; ea.down = L.r_down; ea.sh_gu = L.r_sh_gu; ea.sh_down = L.r_sh_down;
    ea.lists = e->lists; ea.p = P.pbuf[r]; ea.hbuf = e->hbuf; ea.dbuf = e->dbuf; ea.M = T; ea.H = H; ea.I = e->I; ea.topk = topk;
    ea.M_shared = M; ea.shared_row0 = r * M;
    ea.scores = e->scores; ea.sgl = e->sgl; ea.tile_counter = nullptr; ea.err = e->err_flag;
    for (int d = 0; d < R; ++d) ea.peer_dbuf[d] = P.dbuf[d];
    ea.ep_pairs_per_rank = M * topk;
    ea.ep_sig = ra.epd.sig; ea.ep_sig.ticket = e->counters + 2;
    const int local_e = e->ep_e1 - e->ep_e0;
    const int nslots = T * topk < local_e ? T * topk : local_e;
    bool rows_done = false;
    if (T > 8 && local_e <= 256 && e->use_rows && T <= e->cfg.max_rows) {
        launch_rows_prep_plain(P.pbuf[r], H, T, H, e->xq_p, e->sx_p, st);
        ea.xq = e->xq_p; ea.sxq = e->sx_p; ea.csum = e->csum;
        rows_done = launch_expert_rows_gateup(ea, st) && launch_expert_rows_down(ea, st);
    }
    if (!rows_done) {
        launch_expert_gateup(ea, nslots, st, false);
        launch_expert_down(ea, nslots, st, false);       // its last CTA raises the combine flags
    }
    launch_ep_combine(P, e->dbuf + (size_t)T * topk * H, e->scores, e->sgl, M, H, topk, resid, plain_out, layer, e->err_flag, st);
    return SL_OK;
}

// next: the layer after L (nullptr after the last one, where the lm_head follows)
void enqueue_moe(sl_engine* e, const LayerW& L, const LayerW* next, const __half* rows, int ld, bool apply_norm, int M, __half* resid, __half* plain_out) {
    cudaStream_t st = e->stream;
    RouterArgs ra{}; ra.h = rows; ra.ldh = ld; ra.norm_w = apply_norm ? L.post_norm : nullptr; ra.eps = e->cfg.rms_eps;
    ra.router = L.router; ra.shared_gate = L.shared_gate; ra.M = M; ra.H = e->H; ra.E = e->E;
    ra.router_q8 = L.router_q8; ra.router_qs = L.router_qs; ra.router_qb = L.router_qb;
    ra.sg_q8 = L.sg_q8; ra.sg_qs = L.sg_qs; ra.sg_qb = L.sg_qb;
    ra.p = e->p; ra.logits = e->rlogits; ra.sgl = e->sgl;
    ra.topk = e->topk; ra.inds = e->inds; ra.scores = e->scores; ra.lists = e->lists; ra.counter = e->counters + 1;
    ra.group_counter = e->router_groups;
    if (e->ep_step) { enqueue_moe_ep(e, L, ra, M, resid, plain_out); return; }
    ExpertArgs ea{}; ea.gu = L.r_gu; ea.down = L.r_down; ea.sh_gu = L.r_sh_gu; ea.sh_down = L.r_sh_down;
    ea.lists = e->lists; ea.p = e->p; ea.hbuf = e->hbuf; ea.dbuf = e->dbuf; ea.M = M; ea.H = e->H; ea.I = e->I; ea.topk = e->topk;
    ea.scores = e->scores; ea.sgl = e->sgl; ea.resid = resid; ea.out = plain_out; ea.tile_counter = e->tile_counters; ea.err = e->err_flag;
    if (e->use_prefetch) { if (next) pf_q4(ea.pf, 0, next->r_in); else pf_q4(ea.pf, 0, e->r_lm_head, (size_t)24 << 20); }
    int nslots = M * e->topk < e->E ? M * e->topk : e->E;
    ea.slot_sync = e->slot_sync;
    ea.rlogits = e->rlogits; ea.E = e->E; ea.inds_out = e->inds; ea.scores_out = e->scores;
    const bool fused = e->use_fused_experts && !e->hybrid && expert_fused_applicable(ea);   // (prefill mode: one kernel family for any row count)
    // batch-1 decode: the router stops at the logits and the fused expert kernel's CTAs route the row themselves
    ra.no_route = (fused && e->use_route_in_experts) ? 1 : 0;
    ea.route_here = ra.no_route;
    const bool tc_experts = e->hybrid && e->E <= 256 && e->use_rows;      // prefill mode: for any row count (chunk-split invariance)
    const bool rows_experts = !tc_experts && M > 8 && e->E <= 256 && e->use_rows;
    const bool prepared = enqueue_router(e, ra, M, e->use_pdl, rows_experts ? e->xq_p : nullptr, e->sx_p);
    if (fused && launch_expert_fused(ea, st, e->use_pdl)) return;                      // one launch for gate/up + down
    if (tc_experts) {
        // prefill mode: grouped GEMMs on the tensor cores, then the combine kernel
        ea.tile_counter = nullptr;
        if (launch_expert_tc_gateup(ea, st) && launch_expert_tc_down(ea, st)) {
            launch_moe_combine(e->dbuf, e->dbuf + (size_t)M * e->topk * e->H, e->scores, e->sgl, M, e->H, e->topk, resid, plain_out, st);
            return;
        }
        ea.tile_counter = e->tile_counters;
    }
    if (rows_experts || (tc_experts && M > 8)) {
        // many rows: the normed rows are prepared once (by the norm kernel when it ran), the experts run without CTA-wide
        // barriers, the combine is its own kernel
        if (!prepared) launch_rows_prep_plain(e->p, e->H, M, e->H, e->xq_p, e->sx_p, st);
        ea.xq = e->xq_p; ea.sxq = e->sx_p; ea.csum = e->csum; ea.tile_counter = nullptr;
        if (launch_expert_rows_gateup(ea, st) && launch_expert_rows_down(ea, st)) {
            launch_moe_combine(e->dbuf, e->dbuf + (size_t)M * e->topk * e->H, e->scores, e->sgl, M, e->H, e->topk, resid, plain_out, st);
            return;
        }
        ea.tile_counter = e->tile_counters;
    }
    launch_expert_gateup(ea, nslots, st, e->use_pdl);
    launch_expert_down(ea, nslots, st, e->use_pdl);
}

// mixer of one layer: input rows are normed inside (norm_w != nullptr) or already normed
void enqueue_mixer(sl_engine* e, const LayerW& L, const __half* rows, const __half* norm_w, int M, int nsegs,
                   __half* resid, __half* plain_out, const int* row_pos_override) {
    cudaStream_t st = e->stream;
    const sl_config& c = e->cfg;
    DenseArgs d{}; d.err = e->err_flag; d.norm_scratch = e->normed; d.xq = e->use_rows ? e->xq : nullptr; d.sxq = e->sxq; d.q = L.r_in; d.N = (int)L.in_proj.N; d.K = e->H; d.M = M;
    d.x = rows; d.ldx = e->H; d.nw = norm_w; d.eps = c.rms_eps; d.y = e->inproj; d.ldy = (int)L.in_proj.N;
    if (e->use_prefetch) pf_q4(d.pf, 0, L.r_out);
    d.tc = e->hybrid;
    launch_dense(norm_w ? PRO_RMSNORM : PRO_PLAIN, EPI_STORE, d, st, e->use_pdl);
    DenseArgs o{};
    o.err = e->err_flag; o.q = L.r_out; o.N = e->H; o.K = L.out_proj.K; o.M = M;
    o.eps = c.rms_eps; o.y = resid ? resid : plain_out; o.ldy = e->H; o.tc = e->hybrid; o.norm_scratch = e->normed; o.xq = e->use_rows ? e->xq : nullptr; o.sxq = e->sxq;
    if (e->use_prefetch) {
        o.pf.p[0] = L.router; o.pf.bytes[0] = (unsigned)((size_t)e->E * e->H * 2);
        pf_q4(o.pf, 1, L.r_sh_gu);
        pf_q4(o.pf, 3, L.r_sh_down);
    }
    if (!L.is_attn) {
        GdnArgs g{}; g.inproj = e->inproj; g.ld = e->gdn_in; g.conv_w = L.conv_w; g.A_log = L.A_log; g.dt_bias = L.dt_bias;
        g.Hk = c.gdn_k_heads; g.Hv = c.gdn_v_heads; g.eps = c.rms_eps; g.tab = e->tab; g.gdn_index = L.type_index; g.segs = e->segs; g.y = e->mix;
        g.row_seg = e->row_seg; g.qk = e->gdn_qk; g.vc = e->gdn_vc; g.gb = e->gdn_gb;
        // segments of many rows: the state-independent part for all rows side by side, then the bare recurrence (same bits)
        if (e->use_rows && M >= 16) launch_gdn_rows(g, M, nsegs, st);
        else launch_gdn_core(g, nsegs, st, e->use_pdl);
        o.x = e->mix; o.ldx = e->valDim; o.nw = L.gdn_norm; o.nw32 = L.gdn_norm32; o.z = e->inproj + e->convDim; o.ldz = e->gdn_in;
        launch_dense(L.gdn_norm32 ? PRO_NORMGATE32 : PRO_NORMGATE, resid ? EPI_RESID : EPI_STORE, o, st, e->use_pdl);
    } else {
        AttnArgs a{}; a.inproj = e->inproj; a.ld = e->attn_in; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.NH = c.attn_heads; a.KV = c.attn_kv_heads;
        a.eps = c.rms_eps; a.theta = c.rope_theta; a.tab = e->tab; a.attn_index = L.type_index; a.n_attn_layers = e->n_attn > 0 ? e->n_attn : 1;
        a.page_size = c.kv_page_size; a.kv_pool = e->kv_pool; a.segs = e->segs; a.row_seg = e->row_seg; a.row_off = e->row_off;
        a.row_pos_override = row_pos_override; a.qrot = e->qrot; a.part_o = e->part_o; a.part_ml = e->part_ml; a.nsplit = NSPLIT; a.gated = e->mix; a.M = M;
        // a row that is its stream's only row in this call can make its own q/K/V inside the attention kernel;
        // several rows of one stream need every row's K/V in the arena before any of them attends
        // (prefill mode always prepares first and runs the tiled kernel, whatever the row count: chunk-split invariance)
        const bool tiled = e->hybrid && nsegs == 1 && row_pos_override == nullptr && c.kv_page_size % 32 == 0;
        const bool self_prep = !tiled && (M == nsegs) && (row_pos_override == nullptr || M == 1);
        if (!self_prep) launch_attn_prep(a, st);
        // prefill mode, one stream's chunk: the keys are walked once for 64 rows at a time on the tensor cores
        if (!(tiled && launch_attn_prefill(a, nsegs, st)))
            launch_attn_fused(a, self_prep, e->att_counters, st, e->use_pdl && self_prep);
        o.x = e->mix; o.ldx = e->attn_out;
        launch_dense(PRO_PLAIN, resid ? EPI_RESID : EPI_STORE, o, st, e->use_pdl);
    }
}

// all kernels of one call; descriptors / tokens are already on the device
void enqueue_step(sl_engine* e, int M, int nsegs, HeadMode head, bool want_logits) {
    cudaStream_t st = e->stream;
    e->ep_layer_seq = 0;
    launch_embed(e->embed, e->tok_in, M, e->H, e->V, e->h, st);
    for (size_t li = 0; li < e->layers.size(); ++li) {
        const LayerW& L = e->layers[li];
        enqueue_mixer(e, L, e->h, L.in_norm, M, nsegs, e->h, nullptr, nullptr);
        enqueue_moe(e, L, li + 1 < e->layers.size() ? &e->layers[li + 1] : nullptr, e->h, e->H, true, M, e->h, nullptr);
    }
    if (head == HEAD_NORMED) {
        launch_final_norm(e->h, e->final_norm, e->cfg.rms_eps, M, e->H, e->normed, st);
    } else if (head == HEAD_ARGMAX || head == HEAD_LOGITS) {
        DenseArgs d{}; d.q = e->r_lm_head; d.N = e->V; d.K = e->H; d.M = M;
        d.x = e->h; d.ldx = e->H; d.nw = e->final_norm; d.eps = e->cfg.rms_eps;
        d.logits = want_logits ? e->logits : nullptr; d.pval = e->pval; d.pidx = e->pidx; d.out_tok = e->out_tok; d.counter = e->counters + 0;
        launch_dense(PRO_RMSNORM, EPI_ARGMAX, d, st, e->use_pdl);
    }
    StepEndArgs se{}; se.tab = e->tab; se.segs = e->segs; se.nsegs = nsegs; se.M = M;
    se.out_tok = (head == HEAD_ARGMAX || head == HEAD_LOGITS) ? e->out_tok : nullptr;
    se.tok_in = e->tok_in; se.hist = e->hist; se.hist_pos = e->hist_pos; se.hist_cap = e->hist_cap;
    launch_step_end(se, st);
    if (e->ep_step) launch_ep_step_end(e->ep_peers.ctr, st);       // every rank advances its exchange counter once per step
}

// make sure `s` has KV pages for `new_len` positions; uploads new page-table entries
int32_t ensure_pages(sl_stream* s, int new_len) {
    sl_engine* e = s->e;
    if (new_len > s->max_seq_len) return SL_ERR_CAPACITY;
    int need = (new_len + e->cfg.kv_page_size - 1) / e->cfg.kv_page_size;
    int have = (int)s->pages.size();
    if (need <= have) return SL_OK;
    if ((int)e->free_pages.size() < need - have) return SL_ERR_CAPACITY;
    for (int i = have; i < need; ++i) { s->pages.push_back(e->free_pages.back()); e->free_pages.pop_back(); }
    CU(e, cudaMemcpyAsync(e->tab.page_table + (size_t)s->slot * e->tab.max_pages + have, s->pages.data() + have,
                          (size_t)(need - have) * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    // the source is pageable host memory owned by the stream object: make the copy complete before it can change
    CU(e, cudaStreamSynchronize(e->stream));
    return SL_OK;
}

// upload tokens (optional) and row / segment descriptors for a call
int32_t upload_descs(sl_engine* e, const std::vector<SegDesc>& segs, const int32_t* tokens, int M) {
    CU(e, cudaStreamSynchronize(e->stream));    // the pinned staging area may still feed an earlier copy
    int* pin = e->pin_i;
    size_t off = 0;
    int* p_tok = pin + off; off += M;
    int* p_seg = pin + off; off += M;
    int* p_off = pin + off; off += M;
    SegDesc* p_sd = reinterpret_cast<SegDesc*>(pin + off);
    for (size_t si = 0; si < segs.size(); ++si) {
        p_sd[si] = segs[si];
        for (int r = 0; r < segs[si].nrows; ++r) { p_seg[segs[si].row0 + r] = (int)si; p_off[segs[si].row0 + r] = r; }
    }
    if (tokens) {
        memcpy(p_tok, tokens, (size_t)M * sizeof(int));
        CU(e, cudaMemcpyAsync(e->tok_in, p_tok, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    }
    CU(e, cudaMemcpyAsync(e->row_seg, p_seg, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->row_off, p_off, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->segs, p_sd, segs.size() * sizeof(SegDesc), cudaMemcpyHostToDevice, e->stream));
    return SL_OK;
}

// decode-shaped steps (every segment one row) replay a CUDA graph after the first eager run
int32_t enqueue_decode_step(sl_engine* e, int rows) {
    // a single stream's decode step: one launch of the step kernel does the whole token
    if (rows == 1 && !e->ep_step && e->ps_ok && e->use_persistent) {
        profile_launch("k_step_persistent", e->stream, [&] { return launch_step_persistent(e->ps, e->stream); });
        CU(e, cudaGetLastError());
        return SL_OK;
    }
    // (expert-parallel steps contain no collective -- the exchange is this library's own kernels over peer memory --
    // so they are captured like any other step)
    if (!e->use_graph) { enqueue_step(e, rows, rows, HEAD_ARGMAX, false); return e->poisoned ? SL_ERR_CUDA : SL_OK; }
    const int key = rows | (e->ep_step ? (1 << 24) : 0);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        if (e->eager_runs[key]++ == 0) { enqueue_step(e, rows, rows, HEAD_ARGMAX, false); return SL_OK; }
        cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
        CU(e, cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
        const int64_t before = kernel_launch_count();
        enqueue_step(e, rows, rows, HEAD_ARGMAX, false);
        e->graph_kernels[key] = (int)(kernel_launch_count() - before);
        count_launches(-(int64_t)e->graph_kernels[key]);          // the capture itself launched nothing
        CU(e, cudaStreamEndCapture(e->stream, &graph));
        CU(e, cudaGraphInstantiate(&exec, graph, 0));
        cudaGraphDestroy(graph);
        it = e->graphs.emplace(key, exec).first;
    }
    CU(e, cudaGraphLaunch(it->second, e->stream));
    count_launches(e->graph_kernels[key]);
    return SL_OK;
}

int32_t sync_check(sl_engine* e) {
    CU(e, cudaStreamSynchronize(e->stream));
    CU(e, cudaGetLastError());
    // a kernel that gave up a bounded wait went on with whatever it had: the results of this call are not to be trusted
    if (e->err_host && *(volatile unsigned*)e->err_host) {
        char msg[128];
        snprintf(msg, sizeof msg, "a kernel gave up a bounded wait (code %u): results discarded", *(volatile unsigned*)e->err_host);
        return poison_msg(e, msg);
    }
    return SL_OK;
}

int32_t run_single(sl_stream* s, const int32_t* tokens, int M, HeadMode head, bool want_logits) {
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (!tokens || M <= 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    for (int i = 0; i < M; ++i) if (tokens[i] < 0 || tokens[i] >= e->V) return SL_ERR_INVALID;
    if ((rc = ensure_pages(s, s->kv_len + M))) return rc;
    if (want_logits && e->logits_rows < M) {
        __half* lg; if ((rc = dalloc(e, &lg, (size_t)e->cfg.max_rows * e->V))) return rc;
        e->logits = lg; e->logits_rows = e->cfg.max_rows;
    }
    std::vector<SegDesc> segs{SegDesc{s->slot, 0, M, 0}};
    if ((rc = upload_descs(e, segs, tokens, M))) return rc;
    if (M == 1 && head == HEAD_ARGMAX && !want_logits) { if ((rc = enqueue_decode_step(e, 1))) return rc; }
    else enqueue_step(e, M, 1, head, want_logits);
    s->kv_len += M; s->parity ^= 1; s->calls += 1;
    return SL_OK;
}

}  // namespace

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

int32_t sl_engine_destroy(sl_engine* e) {
    if (!e) return SL_ERR_INVALID;
    if (e->ep_comm && g_nccl.ok) { cudaStreamSynchronize(e->stream); g_nccl.CommDestroy((ncclComm_t)e->ep_comm); e->ep_comm = nullptr; }
    for (int d = 0; d < 8; ++d) if (e->ep_mapped[d]) { cudaIpcCloseMemHandle(e->ep_mapped[d]); e->ep_mapped[d] = nullptr; }
    cudaDeviceSynchronize();
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);
    for (void* p : e->allocs) cudaFree(p);
    if (e->pin_i) cudaFreeHost(e->pin_i);
    if (e->err_host) cudaFreeHost(e->err_host);
    if (e->own_stream) cudaStreamDestroy(e->own_stream);
    cudaGetLastError();
    delete e;
    return SL_OK;
}

static int32_t create_common(const sl_config* cfg, sl_engine** out, sl_engine** made) {
    if (!cfg || !out) return SL_ERR_INVALID;
    *out = nullptr;
    if (!config_ok(*cfg)) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    sl_engine* e = new sl_engine();
    e->cfg = *cfg;
    int32_t rc = build_layout(e);
    if (!rc) rc = build_runtime(e);
    if (rc) { sl_engine_destroy(e); return rc; }
    *made = e;
    return SL_OK;
}

int32_t sl_engine_create(const sl_config* cfg, const sl_weight_desc* weights, int32_t n_weights, sl_engine** out) {
    sl_engine* e = nullptr;
    if (!weights || n_weights <= 0) return SL_ERR_INVALID;
    int32_t rc = create_common(cfg, out, &e);
    if (rc) return rc;
    std::map<std::string, bool> seen;
    // the checkpoint's 4-bit embedding ("embed.w/.s/.b") is accepted in place of "embed" and
    // expanded into the fp16 table here
    const sl_weight_desc* eq[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < n_weights; ++i) {
        if (!weights[i].name) continue;
        if (!strcmp(weights[i].name, "embed.w")) eq[0] = &weights[i];
        if (!strcmp(weights[i].name, "embed.s")) eq[1] = &weights[i];
        if (!strcmp(weights[i].name, "embed.b")) eq[2] = &weights[i];
    }
    if (eq[0] || eq[1] || eq[2]) {
        const uint64_t V = (uint64_t)e->V, H = (uint64_t)e->H;
        const uint64_t want[3] = {V * H / 2, V * (H / 64) * 2, V * (H / 64) * 2};
        void* tmp[3] = {nullptr, nullptr, nullptr};
        const void* src[3];
        rc = SL_OK;
        for (int k = 0; k < 3 && !rc; ++k)
            if (!eq[k] || !eq[k]->data || eq[k]->nbytes != want[k]) rc = SL_ERR_INVALID;
        for (int k = 0; k < 3 && !rc; ++k) {
            if (eq[k]->on_device) { src[k] = eq[k]->data; continue; }
            if (cudaMalloc(&tmp[k], want[k]) != cudaSuccess) { cudaGetLastError(); rc = SL_ERR_CAPACITY; break; }
            if (cudaMemcpy(tmp[k], eq[k]->data, want[k], cudaMemcpyHostToDevice) != cudaSuccess) { rc = SL_ERR_CUDA; break; }
            src[k] = tmp[k];
        }
        if (!rc) {
            launch_embed_dequant_q4((const uint32_t*)src[0], (const __half*)src[1], (const __half*)src[2],
                                    const_cast<__half*>(e->embed), e->V, e->H, e->stream);
            if (cudaStreamSynchronize(e->stream) != cudaSuccess || cudaGetLastError() != cudaSuccess) rc = SL_ERR_CUDA;
        }
        for (int k = 0; k < 3; ++k) if (tmp[k]) cudaFree(tmp[k]);
        if (rc) { sl_engine_destroy(e); return rc; }
        seen["embed"] = true;
    }
    // the checkpoint's 8-bit router and shared gate ("L<i>.moe.router.w/.s/.b", "L<i>.moe.shared_gate.w/.s/.b":
    // bytes [E,H] / [H], fp16 scales and biases per 64 inputs) are accepted, per layer, in place of the fp16 pair
    std::vector<char> taken((size_t)n_weights, 0);
    for (int li = 0; li < (int)e->layers.size(); ++li) {
        LayerW& L = e->layers[li];
        const std::string base = "L" + std::to_string(li) + ".moe.";
        const char* suffix[6] = {"router.w", "router.s", "router.b", "shared_gate.w", "shared_gate.s", "shared_gate.b"};
        const uint64_t H = (uint64_t)e->H, E = (uint64_t)e->E;
        const uint64_t want[6] = {E * H, E * (H / 64) * 2, E * (H / 64) * 2, H, (H / 64) * 2, (H / 64) * 2};
        int idx[6]; int found = 0;
        for (int k = 0; k < 6; ++k) {
            idx[k] = -1;
            const std::string nm = base + suffix[k];
            for (int i = 0; i < n_weights; ++i) if (weights[i].name && nm == weights[i].name) { idx[k] = i; ++found; break; }
        }
        if (!found) continue;
        void* dst[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
        rc = (found == 6) ? SL_OK : SL_ERR_INVALID;
        for (int k = 0; k < 6 && !rc; ++k) {
            const sl_weight_desc& d = weights[idx[k]];
            if (!d.data || d.nbytes != want[k]) { rc = SL_ERR_INVALID; break; }
            uint8_t* p8 = nullptr;
            if ((rc = dalloc(e, &p8, (size_t)want[k]))) break;
            if (cudaMemcpy(p8, d.data, want[k], d.on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice) != cudaSuccess) { rc = SL_ERR_CUDA; break; }
            dst[k] = p8; taken[(size_t)idx[k]] = 1;
        }
        if (rc) { sl_engine_destroy(e); return rc; }
        L.router_q8 = (const uint8_t*)dst[0]; L.router_qs = (const __half*)dst[1]; L.router_qb = (const __half*)dst[2];
        L.sg_q8 = (const uint8_t*)dst[3]; L.sg_qs = (const __half*)dst[4]; L.sg_qb = (const __half*)dst[5];
        seen[base + "router"] = true; seen[base + "shared_gate"] = true;
    }
    // "L<i>.gdn.norm.f32" (f32 [128]) in place of "L<i>.gdn.norm": the gated norm of that layer keeps its
    // normed value in f32, as the reference does for an f32 weight (SeedlessFusedVerify.swift:2815-2818)
    for (int i = 0; i < n_weights; ++i) {
        const sl_weight_desc& d = weights[i];
        const size_t len = d.name ? strlen(d.name) : 0;
        if (len < 14 || strcmp(d.name + len - 13, ".gdn.norm.f32")) continue;
        const std::string base(d.name, len - 4);
        auto it = e->tensors.find(base);
        if (it == e->tensors.end()) { sl_engine_destroy(e); return SL_ERR_NOT_FOUND; }
        if (!d.data || d.nbytes != GDN_DV * sizeof(float)) { sl_engine_destroy(e); return SL_ERR_INVALID; }
        float hostw[GDN_DV]; __half hosth[GDN_DV];
        if (cudaMemcpy(hostw, d.data, sizeof(hostw), d.on_device ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost) != cudaSuccess) { sl_engine_destroy(e); return SL_ERR_CUDA; }
        for (int k = 0; k < GDN_DV; ++k) hosth[k] = __float2half_rn(hostw[k]);
        float* w32 = nullptr;
        if ((rc = dalloc(e, &w32, (size_t)GDN_DV))) { sl_engine_destroy(e); return rc; }
        if (cudaMemcpy(w32, hostw, sizeof(hostw), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(it->second.ptr, hosth, sizeof(hosth), cudaMemcpyHostToDevice) != cudaSuccess) { sl_engine_destroy(e); return SL_ERR_CUDA; }
        for (LayerW& L : e->layers) if ((const void*)L.gdn_norm == it->second.ptr) L.gdn_norm32 = w32;
        taken[(size_t)i] = 1; seen[base] = true;
    }
    for (int i = 0; i < n_weights; ++i) {
        const sl_weight_desc& d = weights[i];
        if (&d == eq[0] || &d == eq[1] || &d == eq[2] || taken[(size_t)i]) continue;
        if (d.name && seen.count(d.name) && d.name[0] == 'L') { sl_engine_destroy(e); return SL_ERR_INVALID; }   // both forms given
        if (d.name && seen.count(d.name) && !strcmp(d.name, "embed")) { sl_engine_destroy(e); return SL_ERR_INVALID; }   // both forms given
        auto it = d.name ? e->tensors.find(d.name) : e->tensors.end();
        if (it == e->tensors.end()) { sl_engine_destroy(e); return SL_ERR_NOT_FOUND; }
        if (!d.data || d.nbytes != it->second.bytes) { sl_engine_destroy(e); return SL_ERR_INVALID; }
        if (cudaMemcpy(it->second.ptr, d.data, d.nbytes, d.on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice) != cudaSuccess) {
            sl_engine_destroy(e); return SL_ERR_CUDA;
        }
        seen[d.name] = true;
    }
    if (seen.size() != e->tensors.size()) { sl_engine_destroy(e); return SL_ERR_INVALID; }   // every tensor must be given
    if ((rc = repack_all(e)) || (rc = setup_persistent(e))) { sl_engine_destroy(e); return rc; }
    *out = e;
    return SL_OK;
}

int32_t sl_engine_create_synthetic(const sl_config* cfg, const sl_synth_spec* synth, sl_engine** out) {
    sl_engine* e = nullptr;
    if (!synth) return SL_ERR_INVALID;
    int32_t rc = create_common(cfg, out, &e);
    if (rc) return rc;
    const uint64_t seed = synth->seed;
    cudaStream_t st = e->stream;
    auto has_suffix = [](const std::string& s, const char* suf) { size_t n = strlen(suf); return s.size() >= n && s.compare(s.size() - n, n, suf) == 0; };
    for (auto& kv : e->tensors) {
        const std::string& name = kv.first;
        Tensor& t = kv.second;
        if (has_suffix(name, ".s") || has_suffix(name, ".b")) continue;          // produced together with ".w"
        if (has_suffix(name, ".w")) {
            std::string base = name.substr(0, name.size() - 2);
            Tensor& ts = e->tensors[base + ".s"]; Tensor& tb = e->tensors[base + ".b"];
            int64_t groups = (int64_t)(ts.bytes / 2);
            // the generator indexes groups linearly, so only the total matters: N*K = groups*64
            launch_synth_q4(tensor_seed(seed, base.c_str()), groups, 64, 0.02f, (uint32_t*)t.ptr, (__half*)ts.ptr, (__half*)tb.ptr, st);
        } else if (has_suffix(name, "norm")) {
            launch_synth_f16(tensor_seed(seed, name.c_str()), (int64_t)(t.bytes / 2), 1.0f, synth->norm_jitter, (__half*)t.ptr, st);
        } else if (has_suffix(name, "gdn.conv_w")) {
            launch_synth_f32(tensor_seed(seed, name.c_str()), (int64_t)(t.bytes / 4), 0.0f, synth->conv_std, (float*)t.ptr, st);
        } else if (has_suffix(name, "gdn.A_log") || has_suffix(name, "gdn.dt_bias")) {
            launch_synth_f32(tensor_seed(seed, name.c_str()), (int64_t)(t.bytes / 4), 0.0f, 1.0f, (float*)t.ptr, st);
        } else {   // embed, router, shared_gate: fp16 ~N(0, 0.02)
            launch_synth_f16(tensor_seed(seed, name.c_str()), (int64_t)(t.bytes / 2), 0.0f, 0.02f, (__half*)t.ptr, st);
        }
    }
    if (cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess) { sl_engine_destroy(e); return SL_ERR_CUDA; }
    if ((rc = repack_all(e)) || (rc = setup_persistent(e))) { sl_engine_destroy(e); return rc; }
    *out = e;
    return SL_OK;
}

int32_t sl_engine_set_cuda_stream(sl_engine* e, void* cuda_stream) {
    if (!e) return SL_ERR_INVALID;
    cudaStreamSynchronize(e->stream);
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);    // graphs are tied to the stream they were captured on
    e->graphs.clear(); e->eager_runs.clear();
    e->stream = cuda_stream ? (cudaStream_t)cuda_stream : e->own_stream;
    return SL_OK;
}

int32_t sl_engine_tensor_bytes(sl_engine* e, const char* name, uint64_t* nbytes) {
    if (!e || !name || !nbytes) return SL_ERR_INVALID;
    auto it = e->tensors.find(name);
    if (it == e->tensors.end()) return SL_ERR_NOT_FOUND;
    *nbytes = it->second.bytes;
    return SL_OK;
}
int32_t sl_engine_read_tensor(sl_engine* e, const char* name, void* host_buf, uint64_t nbytes) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!name || !host_buf) return SL_ERR_INVALID;
    auto it = e->tensors.find(name);
    if (it == e->tensors.end()) return SL_ERR_NOT_FOUND;
    if (nbytes != it->second.bytes) return SL_ERR_INVALID;
    CU(e, cudaMemcpy(host_buf, it->second.ptr, nbytes, cudaMemcpyDeviceToHost));
    return SL_OK;
}
const char* sl_last_fault(sl_engine* e) {
    if (!e) return nullptr;
    if (!e->poisoned && e->err_flag) {
        // a kernel whose bounded wait on a bulk copy gave up leaves a mark here instead of hanging
        unsigned flag = 0;
        if (cudaStreamSynchronize(e->stream) == cudaSuccess && (flag = *(volatile unsigned*)e->err_host) != 0) {
            e->poisoned = true; e->fault = "a kernel gave up a bounded wait (code " + std::to_string(flag) + ")";
        }
    }
    return e->poisoned ? e->fault.c_str() : nullptr;
}
int32_t sl_debug_wait_timeout(sl_engine* e) {
    int32_t rc = guard(e); if (rc) return rc;
    launch_wait_probe(e->err_flag, e->stream);
    return SL_OK;
}
int32_t sl_inject_fault(sl_engine* e, int32_t on) { if (!e) return SL_ERR_INVALID; e->inject = on != 0; return SL_OK; }
int64_t sl_engine_launch_count(sl_engine* e) { (void)e; return kernel_launch_count(); }
int32_t sl_engine_use_graphs(sl_engine* e, int32_t on) { if (!e) return SL_ERR_INVALID; e->use_graph = on != 0; return SL_OK; }
int32_t sl_debug_step_timeline(sl_engine* e, int32_t on, uint32_t* out, uint64_t cap_words) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!e->ps_ok) return SL_ERR_NOT_FOUND;
    const size_t words = (size_t)e->ps.geom.G * (e->ps.n_layers + 1) * 24;
    if (on) {
        if (!e->ps_timeline && (rc = dalloc(e, &e->ps_timeline, words))) return rc;
        CU(e, cudaMemsetAsync(e->ps_timeline, 0, words * 4, e->stream));
        e->ps.timeline = e->ps_timeline;
        return (int32_t)e->ps.geom.G;
    }
    e->ps.timeline = nullptr;
    if (out) {
        if (!e->ps_timeline || cap_words < words) return SL_ERR_CAPACITY;
        CU(e, cudaMemcpyAsync(out, e->ps_timeline, words * 4, cudaMemcpyDeviceToHost, e->stream));
        return sync_check(e);
    }
    return SL_OK;
}
int32_t sl_engine_use_persistent(sl_engine* e, int32_t on) {
    if (!e) return SL_ERR_INVALID;
    if (on < 0) return e->ps_ok ? (e->use_persistent ? 1 : 0) : 0;          // query
    e->use_persistent = on != 0;
    return e->ps_ok ? 1 : 0;
}
int32_t sl_profile_start(sl_engine* e) { if (!e) return SL_ERR_INVALID; cudaStreamSynchronize(e->stream); profile_start(); return SL_OK; }
int32_t sl_profile_report(sl_engine* e, char* buf, uint64_t cap) {
    if (!e || !buf) return SL_ERR_INVALID;
    return profile_report(buf, (size_t)cap) < 0 ? SL_ERR_CAPACITY : SL_OK;
}

// ---- streams ----
int32_t sl_stream_create(sl_engine* e, int32_t max_seq_len, sl_stream** out) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!out || max_seq_len <= 0) return SL_ERR_INVALID;
    if (e->free_slots.empty()) return SL_ERR_CAPACITY;
    sl_stream* s = new sl_stream{e, e->free_slots.back(), max_seq_len, 0, 0, {}, 0};
    e->free_slots.pop_back();
    *out = s;
    return sl_stream_reset(s);
}
int32_t sl_stream_destroy(sl_stream* s) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    cudaStreamSynchronize(e->stream);
    for (int pg : s->pages) e->free_pages.push_back(pg);
    e->free_slots.push_back(s->slot);
    delete s;
    return SL_OK;
}
int32_t sl_stream_len(sl_stream* s) { return s ? s->kv_len : SL_ERR_INVALID; }
int32_t sl_stream_reset(sl_stream* s) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    s->kv_len = 0; s->parity = 0;
    for (int pg : s->pages) e->free_pages.push_back(pg);
    s->pages.clear();
    CU(e, cudaMemsetAsync(e->tab.kv_len + s->slot, 0, sizeof(int), e->stream));
    CU(e, cudaMemsetAsync(e->tab.parity + s->slot, 0, sizeof(int), e->stream));
    CU(e, cudaMemsetAsync(e->tab.gdn_state + (size_t)s->slot * e->tab.state_stride_stream, 0, e->tab.state_stride_stream * sizeof(float), e->stream));
    CU(e, cudaMemsetAsync(e->tab.conv_hist + (size_t)s->slot * e->tab.hist_stride_stream, 0, e->tab.hist_stride_stream * sizeof(__half), e->stream));
    return sync_check(e);
}

// ---- forward / step ----
int32_t sl_forward(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_normed_f16) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = run_single(s, tokens, M, HEAD_NORMED, false); if (rc) return rc;
    if (out_normed_f16) CU(e, cudaMemcpyAsync(out_normed_f16, e->normed, (size_t)M * e->H * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_forward_hybrid(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_normed_f16) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    e->hybrid = true;
    int32_t rc = run_single(s, tokens, M, HEAD_NORMED, false);
    e->hybrid = false;
    if (rc) return rc;
    if (out_normed_f16) CU(e, cudaMemcpyAsync(out_normed_f16, e->normed, (size_t)M * e->H * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_hybrid_chunk(sl_engine* e) {
    if (!e) return SL_ERR_INVALID;
    return e->cfg.max_rows < 1024 ? e->cfg.max_rows : 1024;
}
int32_t sl_step_argmax(sl_stream* s, const int32_t* tokens, int32_t M, int32_t* out_tokens) {
    if (!s || !out_tokens) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = run_single(s, tokens, M, HEAD_ARGMAX, false); if (rc) return rc;
    CU(e, cudaMemcpyAsync(out_tokens, e->out_tok, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_step_logits(sl_stream* s, const int32_t* tokens, int32_t M, uint16_t* out_logits_f16) {
    if (!s || !out_logits_f16) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = run_single(s, tokens, M, HEAD_LOGITS, true); if (rc) return rc;
    CU(e, cudaMemcpyAsync(out_logits_f16, e->logits, (size_t)M * e->V * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
// device part shared by the two sampling entry points: logits [M][V] on the device -> three int32 per row on the host
static int32_t drafts_ok(const sl_engine* e, const int32_t* draft, int M) {
    // the kernel reads logits[draft]: anything outside [-1, vocab) would be a read outside the row
    if (draft) for (int i = 0; i < M; ++i) if (draft[i] < -1 || draft[i] >= e->V) return SL_ERR_INVALID;
    return SL_OK;
}
static int32_t sample_rows_device(sl_engine* e, const __half* logits, int M, const int32_t* draft, const float* logit_adj, float inv_t, float top_p,
                                  uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, int32_t* out_full, int32_t* out_resid, int32_t* out_accept) {
    int* d = e->samp_buf;                      // [4][max_rows]: draft, full, resid, accept
    const int R = e->cfg.max_rows;
    if (draft) CU(e, cudaMemcpyAsync(d, draft, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    if (logit_adj) {
        int32_t rc;
        if (!e->adj_buf && (rc = dalloc(e, &e->adj_buf, (size_t)e->V))) return rc;
        CU(e, cudaMemcpyAsync(e->adj_buf, logit_adj, (size_t)e->V * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    }
    launch_sample_rows(logits, logit_adj ? e->adj_buf : nullptr, draft ? d : nullptr, d + R, d + 2 * R, d + 3 * R, M, e->V, inv_t, top_p, seed_lo, seed_hi, base_pos, e->stream);
    if (out_full) CU(e, cudaMemcpyAsync(out_full, d + R, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    if (out_resid) CU(e, cudaMemcpyAsync(out_resid, d + 2 * R, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    if (out_accept) CU(e, cudaMemcpyAsync(out_accept, d + 3 * R, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_step_sample_rows(sl_stream* s, const int32_t* tokens, int32_t M, const int32_t* draft_tokens, const float* logit_adj, float inv_temperature, float top_p,
                            uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, int32_t* out_full, int32_t* out_resid, int32_t* out_accept) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = drafts_ok(e, draft_tokens, M > 0 ? M : 0); if (rc) return rc;
    rc = run_single(s, tokens, M, HEAD_LOGITS, true); if (rc) return rc;
    return sample_rows_device(e, e->logits, M, draft_tokens, logit_adj, inv_temperature, top_p, seed_lo, seed_hi, base_pos, out_full, out_resid, out_accept);
}
int32_t sl_op_sample_rows(sl_engine* e, const uint16_t* logits_f16, int32_t M, const int32_t* draft_tokens, const float* logit_adj, float inv_temperature, float top_p,
                          uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, int32_t* out_full, int32_t* out_resid, int32_t* out_accept) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!logits_f16 || M <= 0) return SL_ERR_INVALID;
    if ((rc = drafts_ok(e, draft_tokens, M))) return rc;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    if (e->logits_rows < M) {
        __half* lg; if ((rc = dalloc(e, &lg, (size_t)e->cfg.max_rows * e->V))) return rc;
        e->logits = lg; e->logits_rows = e->cfg.max_rows;
    }
    CU(e, cudaMemcpyAsync(e->logits, logits_f16, (size_t)M * e->V * 2, cudaMemcpyHostToDevice, e->stream));
    return sample_rows_device(e, e->logits, M, draft_tokens, logit_adj, inv_temperature, top_p, seed_lo, seed_hi, base_pos, out_full, out_resid, out_accept);
}
int32_t sl_chained_enqueue(sl_stream* s, int32_t first, int32_t K) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (K <= 0 || K > e->hist_cap) return SL_ERR_INVALID;
    if (first >= e->V) return SL_ERR_INVALID;
    if ((rc = ensure_pages(s, s->kv_len + K))) return rc;
    std::vector<SegDesc> segs{SegDesc{s->slot, 0, 1, 0}};
    int32_t tok = first;
    if ((rc = upload_descs(e, segs, first >= 0 ? &tok : nullptr, 1))) return rc;
    CU(e, cudaMemsetAsync(e->hist_pos, 0, sizeof(int), e->stream));
    for (int k = 0; k < K; ++k) {
        if ((rc = enqueue_decode_step(e, 1))) return rc;
        s->kv_len += 1; s->parity ^= 1; s->calls += 1;
    }
    return SL_OK;
}
int32_t sl_chained_collect(sl_stream* s, int32_t K, int32_t* out_tokens) {
    if (!s || !out_tokens || K <= 0) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (K > e->hist_cap) return SL_ERR_INVALID;
    CU(e, cudaMemcpyAsync(out_tokens, e->hist, (size_t)K * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_chained_step_argmax(sl_stream* s, int32_t first, int32_t K, int32_t* out_tokens) {
    if (first < 0) return SL_ERR_INVALID;
    int32_t rc = sl_chained_enqueue(s, first, K); if (rc) return rc;
    return sl_chained_collect(s, K, out_tokens);
}

int32_t sl_batch_step_argmax(sl_engine* e, sl_stream* const* streams, const int32_t* tokens, int32_t B, int32_t* out_tokens) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!streams || !tokens || !out_tokens || B <= 0) return SL_ERR_INVALID;
    if (B > e->cfg.max_rows) return SL_ERR_CAPACITY;
    std::vector<SegDesc> segs;
    for (int b = 0; b < B; ++b) {
        if (!streams[b] || streams[b]->e != e) return SL_ERR_INVALID;
        for (int j = 0; j < b; ++j) if (streams[j] == streams[b]) return SL_ERR_INVALID;
        if (tokens[b] < 0 || tokens[b] >= e->V) return SL_ERR_INVALID;
        if ((rc = ensure_pages(streams[b], streams[b]->kv_len + 1))) return rc;
        segs.push_back(SegDesc{streams[b]->slot, b, 1, 0});
    }
    if ((rc = upload_descs(e, segs, tokens, B))) return rc;
    e->ep_step = (e->ep_world > 1 && B == e->ep_rows);    // every rank makes this call with the same B, in lockstep
    rc = enqueue_decode_step(e, B);
    e->ep_step = false;
    if (rc) return rc;
    for (int b = 0; b < B; ++b) { streams[b]->kv_len += 1; streams[b]->parity ^= 1; streams[b]->calls += 1; }
    CU(e, cudaMemcpyAsync(out_tokens, e->out_tok, (size_t)B * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}

// ---- expert-parallel decode (no counterpart in the reference, which runs on one GPU) ----
int32_t sl_ep_unique_id(uint8_t* out128) {
    if (!out128) return SL_ERR_INVALID;
    if (!load_nccl()) return SL_ERR_NOT_FOUND;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return SL_ERR_CUDA;
    memcpy(out128, &id, 128);
    return SL_OK;
}
int32_t sl_ep_init(sl_engine* e, int32_t rank, int32_t world, const uint8_t* id128, int32_t rows_per_rank) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!id128 || world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_rank <= 0) return SL_ERR_INVALID;
    if (e->E % world) return SL_ERR_INVALID;
    if ((int64_t)world * rows_per_rank > e->cfg.max_rows) return SL_ERR_CAPACITY;   // gathered rows use the ordinary buffers
    if (e->ep_comm) return SL_ERR_INVALID;
    if (!load_nccl()) return SL_ERR_NOT_FOUND;
    ncclUniqueId id; memcpy(&id, id128, 128);
    ncclComm_t comm = nullptr;
    NC(e, g_nccl.CommInitRank(&comm, world, id, rank));
    e->ep_comm = comm; e->ep_rank = rank; e->ep_world = world; e->ep_rows = rows_per_rank;
    e->ep_e0 = rank * (e->E / world); e->ep_e1 = e->ep_e0 + e->E / world;
    // The exchange region of this rank: [gathered rows][gathered indices][pair outputs of the local rows][flags, counter].
    // Its CUDA IPC handle goes to every rank through one all-gather on the new communicator (the only collective this
    // mode ever runs); each rank maps every peer's region and from then on talks to it with plain loads and stores.
    const int M = rows_per_rank, T = world * M;
    const size_t b_p = ((size_t)T * e->H * 2 + 255) & ~(size_t)255, b_i = ((size_t)T * e->topk * 4 + 255) & ~(size_t)255;
    const size_t b_d = ((size_t)M * e->topk * e->H * 2 + 255) & ~(size_t)255, b_f = 256;
    unsigned char* region = nullptr;
    if ((rc = dalloc(e, &region, b_p + b_i + b_d + b_f))) return rc;
    CU(e, cudaMemsetAsync(region, 0, b_p + b_i + b_d + b_f, e->stream));
    e->ep_region = region;
    cudaIpcMemHandle_t mine;
    CU(e, cudaIpcGetMemHandle(&mine, region));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    unsigned char* hbuf = nullptr;
    if ((rc = dalloc(e, &hbuf, (size_t)64 * world))) return rc;
    CU(e, cudaMemcpyAsync(hbuf + 64 * rank, &mine, 64, cudaMemcpyHostToDevice, e->stream));
    NC(e, g_nccl.AllGather(hbuf + 64 * rank, hbuf, 64, ncclUint8, comm, e->stream));
    std::vector<cudaIpcMemHandle_t> all((size_t)world);
    CU(e, cudaMemcpyAsync(all.data(), hbuf, (size_t)64 * world, cudaMemcpyDeviceToHost, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    EpPeers& P = e->ep_peers;
    P.world = world; P.rank = rank;
    for (int d = 0; d < world; ++d) {
        unsigned char* base = region;
        if (d != rank) {
            void* mapped = nullptr;
            CU(e, cudaIpcOpenMemHandle(&mapped, all[(size_t)d], cudaIpcMemLazyEnablePeerAccess));
            e->ep_mapped[d] = mapped; base = (unsigned char*)mapped;
        }
        P.pbuf[d] = (__half*)base; P.ibuf[d] = (int*)(base + b_p); P.dbuf[d] = (__half*)(base + b_p + b_i);
        P.flags[d] = (unsigned*)(base + b_p + b_i + b_d);
    }
    P.ctr = (unsigned*)(region + b_p + b_i + b_d) + 32;
    return SL_OK;
}

// ---- snapshot / rollback ----
static int32_t push_len_parity(sl_stream* s) {
    sl_engine* e = s->e;
    int v[2] = {s->kv_len, s->parity};
    CU(e, cudaMemcpyAsync(e->tab.kv_len + s->slot, &v[0], sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->tab.parity + s->slot, &v[1], sizeof(int), cudaMemcpyHostToDevice, e->stream));
    return sync_check(e);
}
int32_t sl_snapshot(sl_stream* s, sl_snap* out) {
    if (!s || !out) return SL_ERR_INVALID;
    out->kv_len = s->kv_len; out->parity = s->parity; out->valid = 1; out->calls = s->calls;
    return SL_OK;
}
int32_t sl_rollback_one_step(sl_stream* s, const sl_snap* snap) {
    if (!s || !snap || !snap->valid) return SL_ERR_INVALID;
    int32_t rc = guard(s->e); if (rc) return rc;
    if (snap->kv_len > s->kv_len) return SL_ERR_INVALID;
    if (snap->kv_len == s->kv_len) return SL_OK;           // nothing ran since the snapshot
    // exactly one call may have run: after two the other ping-pong side no longer holds the old state, and after
    // any odd number the parity alone would not tell
    if (s->calls != snap->calls + 1 || s->parity == snap->parity) return SL_ERR_INVALID;
    s->kv_len = snap->kv_len; s->parity = snap->parity; s->calls = snap->calls;
    return push_len_parity(s);
}
static float* cur_state(sl_stream* s) { return s->e->tab.gdn_state + (size_t)s->slot * s->e->tab.state_stride_stream + (size_t)s->parity * s->e->tab.state_stride_side; }
static __half* cur_hist(sl_stream* s) { return s->e->tab.conv_hist + (size_t)s->slot * s->e->tab.hist_stride_stream + (size_t)s->parity * s->e->tab.hist_stride_side; }

int32_t sl_full_snapshot(sl_stream* s, sl_fullsnap** out) {
    if (!s || !out) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    sl_fullsnap* f = new sl_fullsnap{s->kv_len, nullptr, nullptr};
    size_t sb = e->tab.state_stride_side * sizeof(float), hb = e->tab.hist_stride_side * sizeof(__half);
    if (cudaMalloc(&f->state, sb) != cudaSuccess || cudaMalloc(&f->hist, hb) != cudaSuccess) {
        cudaGetLastError(); if (f->state) cudaFree(f->state); delete f; return SL_ERR_CAPACITY;
    }
    CU(e, cudaMemcpyAsync(f->state, cur_state(s), sb, cudaMemcpyDeviceToDevice, e->stream));
    CU(e, cudaMemcpyAsync(f->hist, cur_hist(s), hb, cudaMemcpyDeviceToDevice, e->stream));
    rc = sync_check(e);
    if (rc) { cudaFree(f->state); cudaFree(f->hist); delete f; return rc; }
    *out = f;
    return SL_OK;
}
int32_t sl_full_restore(sl_stream* s, const sl_fullsnap* f) {
    if (!s || !f) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (f->kv_len > s->kv_len) return SL_ERR_INVALID;      // KV is append-only: only rewinds are possible
    size_t sb = e->tab.state_stride_side * sizeof(float), hb = e->tab.hist_stride_side * sizeof(__half);
    CU(e, cudaMemcpyAsync(cur_state(s), f->state, sb, cudaMemcpyDeviceToDevice, e->stream));
    CU(e, cudaMemcpyAsync(cur_hist(s), f->hist, hb, cudaMemcpyDeviceToDevice, e->stream));
    s->kv_len = f->kv_len;
    return push_len_parity(s);
}
int32_t sl_fullsnap_free(sl_fullsnap* f) {
    if (!f) return SL_ERR_INVALID;
    cudaFree(f->state); cudaFree(f->hist); delete f;
    return SL_OK;
}

// ---- "QWS1" blob ----
int32_t sl_state_size(sl_stream* s, uint64_t* nbytes) {
    if (!s || !nbytes) return SL_ERR_INVALID;
    sl_engine* e = s->e; const sl_config& c = e->cfg;
    uint64_t n = 12;
    for (const LayerW& L : e->layers) {
        n += 4;
        if (L.is_attn) n += 12 + 2ull * c.attn_kv_heads * s->kv_len * ATT_D * 2;
        else n += 8 + (uint64_t)(CONV_K - 1) * e->convDim * 2 + (uint64_t)c.gdn_v_heads * GDN_DV * GDN_DK * 4;
    }
    *nbytes = n;
    return SL_OK;
}
// copy positions [0,len) of (layer, K|V, head) between the paged arena and a contiguous host run
static int32_t kv_copy(sl_stream* s, int attn_index, int which, int kvh, int len, uint8_t* host, bool to_host) {
    sl_engine* e = s->e; const sl_config& c = e->cfg;
    size_t page_elems = (size_t)e->n_attn * 2 * c.attn_kv_heads * c.kv_page_size * ATT_D;
    for (int p0 = 0; p0 < len; p0 += c.kv_page_size) {
        int n = len - p0 < c.kv_page_size ? len - p0 : c.kv_page_size;
        __half* dev = e->kv_pool + (size_t)s->pages[p0 / c.kv_page_size] * page_elems +
                      (((size_t)attn_index * 2 + which) * c.attn_kv_heads + kvh) * c.kv_page_size * ATT_D;
        uint8_t* hp = host + (size_t)p0 * ATT_D * 2;
        if (to_host) CU(e, cudaMemcpyAsync(hp, dev, (size_t)n * ATT_D * 2, cudaMemcpyDeviceToHost, e->stream));
        else CU(e, cudaMemcpyAsync(dev, hp, (size_t)n * ATT_D * 2, cudaMemcpyHostToDevice, e->stream));
    }
    return SL_OK;
}
int32_t sl_state_save(sl_stream* s, void* buf, uint64_t nbytes) {
    if (!s || !buf) return SL_ERR_INVALID;
    sl_engine* e = s->e; const sl_config& c = e->cfg;
    int32_t rc = guard(e); if (rc) return rc;
    uint64_t need; sl_state_size(s, &need);
    if (nbytes < need) return SL_ERR_CAPACITY;
    uint8_t* p = (uint8_t*)buf;
    auto u32 = [&](uint32_t v) { memcpy(p, &v, 4); p += 4; };
    u32(0x31535751u); u32(1); u32((uint32_t)c.n_layers);
    for (const LayerW& L : e->layers) {
        if (L.is_attn) {
            u32(1); u32(c.attn_kv_heads); u32(ATT_D); u32(s->kv_len);
            for (int which = 0; which < 2; ++which)
                for (int hh = 0; hh < c.attn_kv_heads; ++hh) {
                    if ((rc = kv_copy(s, L.type_index, which, hh, s->kv_len, p, true))) return rc;
                    p += (size_t)s->kv_len * ATT_D * 2;
                }
        } else {
            size_t cc = e->tab.hist_stride_layer, sc = e->tab.state_stride_layer;
            u32(2); u32((uint32_t)cc); u32((uint32_t)sc);
            CU(e, cudaMemcpyAsync(p, cur_hist(s) + (size_t)L.type_index * cc, cc * 2, cudaMemcpyDeviceToHost, e->stream)); p += cc * 2;
            CU(e, cudaMemcpyAsync(p, cur_state(s) + (size_t)L.type_index * sc, sc * 4, cudaMemcpyDeviceToHost, e->stream)); p += sc * 4;
        }
    }
    return sync_check(e);
}
int32_t sl_state_restore(sl_stream* s, const void* buf, uint64_t nbytes) {
    if (!s || !buf) return SL_ERR_INVALID;
    sl_engine* e = s->e; const sl_config& c = e->cfg;
    int32_t rc = guard(e); if (rc) return rc;
    const uint8_t* b = (const uint8_t*)buf;
    // pass 1: validate the whole blob before touching the stream
    uint64_t off = 0; bool ok = true;
    auto u32 = [&]() -> uint32_t { if (off + 4 > nbytes) { ok = false; return 0; } uint32_t v; memcpy(&v, b + off, 4); off += 4; return v; };
    if (u32() != 0x31535751u || u32() != 1u || u32() != (uint32_t)c.n_layers || !ok) return SL_ERR_FORMAT;
    int len = -1;
    for (const LayerW& L : e->layers) {
        uint32_t flags = u32(); if (!ok) return SL_ERR_FORMAT;
        if (flags != (L.is_attn ? 1u : 2u)) return SL_ERR_FORMAT;
        if (L.is_attn) {
            uint32_t kv = u32(), d = u32(), l = u32(); if (!ok) return SL_ERR_FORMAT;
            if (kv != (uint32_t)c.attn_kv_heads || d != (uint32_t)ATT_D || (int)l > s->max_seq_len) return SL_ERR_FORMAT;
            if (len >= 0 && (int)l != len) return SL_ERR_FORMAT;
            len = (int)l;
            off += 2ull * kv * l * d * 2;
        } else {
            uint32_t cc = u32(), sc = u32(); if (!ok) return SL_ERR_FORMAT;
            if (cc != (uint32_t)e->tab.hist_stride_layer || sc != (uint32_t)e->tab.state_stride_layer) return SL_ERR_FORMAT;
            off += (uint64_t)cc * 2 + (uint64_t)sc * 4;
        }
        if (off > nbytes) return SL_ERR_FORMAT;
    }
    if (off != nbytes) return SL_ERR_FORMAT;
    if (len < 0) len = 0;
    if ((rc = ensure_pages(s, len))) return rc;
    // pass 2: copy
    off = 12;
    for (const LayerW& L : e->layers) {
        off += 4;
        if (L.is_attn) {
            off += 12;
            for (int which = 0; which < 2; ++which)
                for (int hh = 0; hh < c.attn_kv_heads; ++hh) {
                    if ((rc = kv_copy(s, L.type_index, which, hh, len, const_cast<uint8_t*>(b + off), false))) return rc;
                    off += (size_t)len * ATT_D * 2;
                }
        } else {
            size_t cc = e->tab.hist_stride_layer, sc = e->tab.state_stride_layer;
            off += 8;
            CU(e, cudaMemcpyAsync(cur_hist(s) + (size_t)L.type_index * cc, b + off, cc * 2, cudaMemcpyHostToDevice, e->stream)); off += cc * 2;
            CU(e, cudaMemcpyAsync(cur_state(s) + (size_t)L.type_index * sc, b + off, sc * 4, cudaMemcpyHostToDevice, e->stream)); off += sc * 4;
        }
    }
    s->kv_len = len;
    return push_len_parity(s);
}

// ---- single operators ----
int32_t sl_op_repack_q4_device(const void* w_dev, const void* s_dev, const void* b_dev, int32_t K, int32_t N,
                               void* wr_dev, void* sr_dev, void* cuda_stream) {
    if (!w_dev || !s_dev || !b_dev || !wr_dev || !sr_dev) return SL_ERR_INVALID;
    if (N <= 0 || K <= 0 || N % 16 || K % 256 || K > 4096) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    Q4W q; q.w = (const uint32_t*)w_dev; q.s = (const __half*)s_dev; q.b = (const __half*)b_dev; q.N = N; q.K = K;
    launch_repack_q4(q, nullptr, (uint4*)wr_dev, (uint4*)sr_dev, (cudaStream_t)cuda_stream);
    return cudaGetLastError() == cudaSuccess ? SL_OK : SL_ERR_CUDA;
}
int32_t sl_op_qmm4_device(const void* x_dev, const void* wr_dev, const void* sr_dev,
                          int32_t M, int32_t K, int32_t N, void* y_dev, void* cuda_stream) {
    if (!x_dev || !wr_dev || !sr_dev || !y_dev) return SL_ERR_INVALID;
    if (M <= 0 || N <= 0 || K <= 0 || N % 16 || !k_ok(K)) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    DenseArgs a{}; a.q.wr = (const uint4*)wr_dev; a.q.sr = (const uint4*)sr_dev; a.q.tiles = N / 16; a.q.K = K; a.N = N; a.K = K; a.M = M;
    a.x = (const __half*)x_dev; a.ldx = K; a.y = (__half*)y_dev; a.ldy = N;
    launch_dense(PRO_PLAIN, EPI_STORE, a, (cudaStream_t)cuda_stream, false);
    return cudaGetLastError() == cudaSuccess ? SL_OK : SL_ERR_CUDA;
}
int32_t sl_op_lm_head_argmax_static(const void* x_dev, const void* wr_dev, const void* sr_dev,
                                    int32_t M, int32_t K, int32_t N, int32_t* out_tokens_dev, void* cuda_stream) {
    if (!x_dev || !wr_dev || !sr_dev || !out_tokens_dev) return SL_ERR_INVALID;
    if (M <= 0 || N <= 0 || K <= 0 || N % 16 || !k_ok(K)) return SL_ERR_INVALID;
    if (M > head_static_max_rows()) {
        fprintf(stderr, "sl_op_lm_head_argmax_static: M = %d rows exceed the fixed scratch array's limit of %d rows per call\n",
                (int)M, head_static_max_rows());
        return SL_ERR_CAPACITY;
    }
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    DenseArgs a{}; a.q.wr = (const uint4*)wr_dev; a.q.sr = (const uint4*)sr_dev; a.q.tiles = N / 16; a.q.K = K; a.N = N; a.K = K; a.M = M;
    a.x = (const __half*)x_dev; a.ldx = K; a.out_tok = out_tokens_dev;
    int err = launch_head_static(a, (cudaStream_t)cuda_stream);
    if (err != 0) {
        fprintf(stderr, "sl_op_lm_head_argmax_static: CUDA error %d (%s)\n", err, cudaGetErrorString((cudaError_t)err));
        return SL_ERR_CUDA;
    }
    return SL_OK;
}
int32_t sl_op_qmm4_tc_device(const void* x_dev, const void* wr_dev, const void* sr_dev,
                             int32_t M, int32_t K, int32_t N, void* y_dev, void* cuda_stream) {
    if (!x_dev || !wr_dev || !sr_dev || !y_dev) return SL_ERR_INVALID;
    if (M <= 0 || N <= 0 || K <= 0 || N % 16 || !k_ok(K)) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    Q4R q{}; q.wr = (const uint4*)wr_dev; q.sr = (const uint4*)sr_dev; q.tiles = N / 16; q.K = K;
    int err = launch_gemm_tc(q, N, K, M, (const __half*)x_dev, K, (__half*)y_dev, N, false, nullptr, (cudaStream_t)cuda_stream);
    return err == 0 ? SL_OK : SL_ERR_CUDA;
}
int32_t sl_op_qmm4(const uint16_t* x, const uint32_t* w, const uint16_t* sc, const uint16_t* bi, int32_t M, int32_t K, int32_t N, uint16_t* y) {
    if (!x || !w || !sc || !bi || !y) return SL_ERR_INVALID;
    if (M <= 0 || N <= 0 || K <= 0 || N % 16 || !k_ok(K)) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    void *dx = nullptr, *dw = nullptr, *ds = nullptr, *db = nullptr, *dy = nullptr, *dwr = nullptr, *dsr = nullptr;
    size_t bx = (size_t)M * K * 2, bw = (size_t)N * K / 2, bs = (size_t)N * K / 64 * 2, by = (size_t)M * N * 2;
    size_t bwr = (size_t)(N / 16) * q4r_w_uint4(K) * 16, bsr = (size_t)(N / 16) * q4r_s_uint4(K) * 16;
    int32_t rc = SL_ERR_CUDA;
    if (cudaMalloc(&dx, bx) == cudaSuccess && cudaMalloc(&dw, bw) == cudaSuccess && cudaMalloc(&ds, bs) == cudaSuccess &&
        cudaMalloc(&db, bs) == cudaSuccess && cudaMalloc(&dy, by) == cudaSuccess && cudaMalloc(&dwr, bwr) == cudaSuccess && cudaMalloc(&dsr, bsr) == cudaSuccess) {
        cudaMemcpy(dx, x, bx, cudaMemcpyHostToDevice); cudaMemcpy(dw, w, bw, cudaMemcpyHostToDevice);
        cudaMemcpy(ds, sc, bs, cudaMemcpyHostToDevice); cudaMemcpy(db, bi, bs, cudaMemcpyHostToDevice);
        rc = sl_op_repack_q4_device(dw, ds, db, K, N, dwr, dsr, nullptr);
        if (rc == SL_OK) rc = sl_op_qmm4_device(dx, dwr, dsr, M, K, N, dy, nullptr);
        if (rc == SL_OK && cudaMemcpy(y, dy, by, cudaMemcpyDeviceToHost) != cudaSuccess) rc = SL_ERR_CUDA;
    }
    cudaFree(dx); cudaFree(dw); cudaFree(ds); cudaFree(db); cudaFree(dy); cudaFree(dwr); cudaFree(dsr);
    cudaGetLastError();
    return rc;
}
int32_t sl_op_quantize_q4(const uint16_t* w, int64_t N, int64_t K, uint32_t* packed, uint16_t* sc, uint16_t* bi) {
    if (!w || !packed || !sc || !bi || N <= 0 || K <= 0 || K % 64) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    void *dw = nullptr, *dp = nullptr, *ds = nullptr, *db = nullptr;
    size_t bw = (size_t)N * K * 2, bp = (size_t)N * K / 2, bs = (size_t)N * K / 64 * 2;
    int32_t rc = SL_ERR_CUDA;
    if (cudaMalloc(&dw, bw) == cudaSuccess && cudaMalloc(&dp, bp) == cudaSuccess && cudaMalloc(&ds, bs) == cudaSuccess && cudaMalloc(&db, bs) == cudaSuccess) {
        cudaMemcpy(dw, w, bw, cudaMemcpyHostToDevice);
        launch_quantize_q4((const __half*)dw, N, K, (uint32_t*)dp, (__half*)ds, (__half*)db, 0);
        if (cudaMemcpy(packed, dp, bp, cudaMemcpyDeviceToHost) == cudaSuccess && cudaMemcpy(sc, ds, bs, cudaMemcpyDeviceToHost) == cudaSuccess &&
            cudaMemcpy(bi, db, bs, cudaMemcpyDeviceToHost) == cudaSuccess) rc = SL_OK;
    }
    cudaFree(dw); cudaFree(dp); cudaFree(ds); cudaFree(db);
    cudaGetLastError();
    return rc;
}
int32_t sl_op_moe_block(sl_engine* e, int32_t layer, const uint16_t* x, int32_t M, uint16_t* out, int32_t* inds, uint16_t* scores) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!x || !out || layer < 0 || layer >= e->cfg.n_layers || M <= 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    CU(e, cudaMemcpyAsync(e->opx, x, (size_t)M * e->H * 2, cudaMemcpyHostToDevice, e->stream));
    enqueue_moe(e, e->layers[layer], nullptr, e->opx, e->H, false, M, nullptr, e->opy);
    CU(e, cudaMemcpyAsync(out, e->opy, (size_t)M * e->H * 2, cudaMemcpyDeviceToHost, e->stream));
    if (inds) CU(e, cudaMemcpyAsync(inds, e->inds, (size_t)M * e->topk * 4, cudaMemcpyDeviceToHost, e->stream));
    if (scores) CU(e, cudaMemcpyAsync(scores, e->scores, (size_t)M * e->topk * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_op_mixer(sl_stream* s, int32_t layer, const uint16_t* x, int32_t M, int32_t pos0, uint16_t* out) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (!x || !out || layer < 0 || layer >= e->cfg.n_layers || M <= 0 || pos0 < 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    if ((rc = ensure_pages(s, pos0 + M))) return rc;
    std::vector<SegDesc> segs{SegDesc{s->slot, 0, M, 0}};
    if ((rc = upload_descs(e, segs, nullptr, M))) return rc;
    std::vector<int> pos(M);
    for (int i = 0; i < M; ++i) pos[i] = pos0 + i;
    CU(e, cudaMemcpyAsync(e->row_pos, pos.data(), (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->opx, x, (size_t)M * e->H * 2, cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    const LayerW& L = e->layers[layer];
    enqueue_mixer(e, L, e->opx, nullptr, M, 1, nullptr, e->opy, e->row_pos);
    if (!L.is_attn) {
        // the GDN core wrote the other ping-pong side; this operator advances only this layer, so copy it back
        size_t sc = e->tab.state_stride_layer, cc = e->tab.hist_stride_layer;
        float* cur = cur_state(s) + (size_t)L.type_index * sc;
        float* oth = e->tab.gdn_state + (size_t)s->slot * e->tab.state_stride_stream + (size_t)(s->parity ^ 1) * e->tab.state_stride_side + (size_t)L.type_index * sc;
        __half* curh = cur_hist(s) + (size_t)L.type_index * cc;
        __half* othh = e->tab.conv_hist + (size_t)s->slot * e->tab.hist_stride_stream + (size_t)(s->parity ^ 1) * e->tab.hist_stride_side + (size_t)L.type_index * cc;
        CU(e, cudaMemcpyAsync(cur, oth, sc * 4, cudaMemcpyDeviceToDevice, e->stream));
        CU(e, cudaMemcpyAsync(curh, othh, cc * 2, cudaMemcpyDeviceToDevice, e->stream));
    }
    CU(e, cudaMemcpyAsync(out, e->opy, (size_t)M * e->H * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_op_read_kv(sl_stream* s, int32_t layer, int32_t pos0, int32_t n, uint16_t* out_k_f16, uint16_t* out_v_f16) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e; const sl_config& c = e->cfg;
    int32_t rc = guard(e); if (rc) return rc;
    if (layer < 0 || layer >= c.n_layers || !e->layers[layer].is_attn || pos0 < 0 || n <= 0) return SL_ERR_INVALID;
    if ((pos0 + n + c.kv_page_size - 1) / c.kv_page_size > (int)s->pages.size()) return SL_ERR_CAPACITY;
    const size_t page_elems = (size_t)e->n_attn * 2 * c.attn_kv_heads * c.kv_page_size * ATT_D;
    for (int which = 0; which < 2; ++which) {
        uint16_t* out = which ? out_v_f16 : out_k_f16;
        if (!out) continue;
        for (int hh = 0; hh < c.attn_kv_heads; ++hh)
            for (int i = 0; i < n; ++i) {
                const int pos = pos0 + i;
                const __half* dev = e->kv_pool + (size_t)s->pages[pos / c.kv_page_size] * page_elems +
                                    ((((size_t)e->layers[layer].type_index * 2 + which) * c.attn_kv_heads + hh) * c.kv_page_size + pos % c.kv_page_size) * ATT_D;
                CU(e, cudaMemcpyAsync(out + ((size_t)hh * n + i) * ATT_D, dev, ATT_D * 2, cudaMemcpyDeviceToHost, e->stream));
            }
    }
    return sync_check(e);
}
int32_t sl_op_layer(sl_stream* s, int32_t layer, const uint16_t* h_in, int32_t M, int32_t pos0, uint16_t* h_out) {
    if (!s) return SL_ERR_INVALID;
    sl_engine* e = s->e;
    int32_t rc = guard(e); if (rc) return rc;
    if (!h_in || !h_out || layer < 0 || layer >= e->cfg.n_layers || M <= 0 || pos0 < 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    if ((rc = ensure_pages(s, pos0 + M))) return rc;
    std::vector<SegDesc> segs{SegDesc{s->slot, 0, M, 0}};
    if ((rc = upload_descs(e, segs, nullptr, M))) return rc;
    std::vector<int> pos(M);
    for (int i = 0; i < M; ++i) pos[i] = pos0 + i;
    CU(e, cudaMemcpyAsync(e->row_pos, pos.data(), (size_t)M * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->h, h_in, (size_t)M * e->H * 2, cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    const LayerW& L = e->layers[layer];
    enqueue_mixer(e, L, e->h, L.in_norm, M, 1, e->h, nullptr, e->row_pos);
    enqueue_moe(e, L, nullptr, e->h, e->H, true, M, e->h, nullptr);
    if (!L.is_attn) {
        size_t sc = e->tab.state_stride_layer, cc = e->tab.hist_stride_layer;
        float* cur = cur_state(s) + (size_t)L.type_index * sc;
        float* oth = e->tab.gdn_state + (size_t)s->slot * e->tab.state_stride_stream + (size_t)(s->parity ^ 1) * e->tab.state_stride_side + (size_t)L.type_index * sc;
        __half* curh = cur_hist(s) + (size_t)L.type_index * cc;
        __half* othh = e->tab.conv_hist + (size_t)s->slot * e->tab.hist_stride_stream + (size_t)(s->parity ^ 1) * e->tab.hist_stride_side + (size_t)L.type_index * cc;
        CU(e, cudaMemcpyAsync(cur, oth, sc * 4, cudaMemcpyDeviceToDevice, e->stream));
        CU(e, cudaMemcpyAsync(curh, othh, cc * 2, cudaMemcpyDeviceToDevice, e->stream));
    }
    CU(e, cudaMemcpyAsync(h_out, e->h, (size_t)M * e->H * 2, cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_op_head(sl_engine* e, const uint16_t* h_rows, int32_t M, uint16_t* out_logits, int32_t* out_tokens) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!h_rows || M <= 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    if (out_logits && e->logits_rows < M) {
        __half* lg; if ((rc = dalloc(e, &lg, (size_t)e->cfg.max_rows * e->V))) return rc;
        e->logits = lg; e->logits_rows = e->cfg.max_rows;
    }
    CU(e, cudaMemcpyAsync(e->opx, h_rows, (size_t)M * e->H * 2, cudaMemcpyHostToDevice, e->stream));
    DenseArgs d{}; d.q = e->r_lm_head; d.N = e->V; d.K = e->H; d.M = M;
    d.x = e->opx; d.ldx = e->H; d.nw = e->final_norm; d.eps = e->cfg.rms_eps;
    d.logits = out_logits ? e->logits : nullptr; d.pval = e->pval; d.pidx = e->pidx; d.out_tok = e->out_tok; d.counter = e->counters + 0;
    launch_dense(PRO_RMSNORM, EPI_ARGMAX, d, e->stream, false);
    if (out_logits) CU(e, cudaMemcpyAsync(out_logits, e->logits, (size_t)M * e->V * 2, cudaMemcpyDeviceToHost, e->stream));
    if (out_tokens) CU(e, cudaMemcpyAsync(out_tokens, e->out_tok, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}
int32_t sl_op_lm_head(sl_engine* e, const uint16_t* normed, int32_t M, uint16_t* out_logits, int32_t* out_tokens) {
    int32_t rc = guard(e); if (rc) return rc;
    if (!normed || M <= 0) return SL_ERR_INVALID;
    if (M > e->cfg.max_rows) return SL_ERR_CAPACITY;
    if (out_logits && e->logits_rows < M) {
        __half* lg; if ((rc = dalloc(e, &lg, (size_t)e->cfg.max_rows * e->V))) return rc;
        e->logits = lg; e->logits_rows = e->cfg.max_rows;
    }
    CU(e, cudaMemcpyAsync(e->opx, normed, (size_t)M * e->H * 2, cudaMemcpyHostToDevice, e->stream));
    DenseArgs d{}; d.q = e->r_lm_head; d.N = e->V; d.K = e->H; d.M = M;
    d.x = e->opx; d.ldx = e->H; d.logits = out_logits ? e->logits : nullptr; d.pval = e->pval; d.pidx = e->pidx; d.out_tok = e->out_tok; d.counter = e->counters + 0;
    launch_dense(PRO_PLAIN, EPI_ARGMAX, d, e->stream, false);
    if (out_logits) CU(e, cudaMemcpyAsync(out_logits, e->logits, (size_t)M * e->V * 2, cudaMemcpyDeviceToHost, e->stream));
    if (out_tokens) CU(e, cudaMemcpyAsync(out_tokens, e->out_tok, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return sync_check(e);
}

// ---- synthetic data helpers ----
int32_t sl_synth_tokens(uint64_t seed, const char* name, int64_t n, int32_t vocab, int32_t* out) {
    if (!name || !out || n < 0 || vocab <= 0) return SL_ERR_INVALID;
    host_synth_tokens(tensor_seed(seed, name), n, vocab, out);
    return SL_OK;
}
int32_t sl_synth_f16(uint64_t seed, const char* name, int64_t n, float mean, float std, uint16_t* out) {
    if (!name || !out || n <= 0) return SL_ERR_INVALID;
    if (!device_ok()) return SL_ERR_NO_DEVICE;
    void* d = nullptr;
    if (cudaMalloc(&d, (size_t)n * 2) != cudaSuccess) { cudaGetLastError(); return SL_ERR_CUDA; }
    launch_synth_f16(tensor_seed(seed, name), n, mean, std, (__half*)d, 0);
    int32_t rc = cudaMemcpy(out, d, (size_t)n * 2, cudaMemcpyDeviceToHost) == cudaSuccess ? SL_OK : SL_ERR_CUDA;
    cudaFree(d); cudaGetLastError();
    return rc;
}

}  // extern "C"
