// step_persistent.cu -- batch-1 decode: one whole token (embedding, every layer, lm_head, argmax, cache
// bookkeeping) in ONE cooperative kernel launch, one CTA per multiprocessor.
//
// Why.  A decode token reads 1.7 GB of weights exactly once, so the floor is HBM time; what the
// kernel-per-phase assembly loses is everything else: each of its ~200 launches asks for its weights when
// it starts, waits for them, computes, and leaves HBM idle across the boundary.  Here the weights never
// wait for the activations:
//   * every CTA owns a ring of weight slots in shared memory (2304 B each: one 16-row x 256-input
//     "unit" of the fragment-major layout, gemv.cuh).  A producer warp walks the CTA's static schedule
//     for the WHOLE token -- this layer's in-projection units, state rows, out-projection, router rows,
//     shared expert, then the next layer's, ... the lm_head -- and issues bulk asynchronous copies
//     (cp.async.bulk + mbarrier, no multicast) as far ahead as the ring has room.  The ring is ordered by
//     consumption but filled out of order: the routed experts' units, whose addresses exist only after
//     the router has run, are issued by a second producer warp the moment the routing is known, while
//     the first one is already fetching the next layer.
//   * the phases of a layer meet through tiny activation vectors in global memory (L2), written and read
//     with a flag-in-data protocol: every 16-byte line carries 8 bytes of data and two copies of the
//     step's sequence number, the reader polls the line itself.  No grid-wide barrier, no fence: a phase
//     starts on an SM as soon as the lines it needs have landed.
// Every wait (ring slot, exchange line) is bounded by a cycle budget; the first one that runs out sets an
// abort flag that makes every later wait in the grid return at once, and the host sees the error word.
//
// The arithmetic is the per-phase kernels' arithmetic, function for function (gemv.cuh, mixer_math.cuh,
// route_row_warp): the same per-unit tensor-core products, the same ascending-slice sums, the same norm /
// softmax / recurrence order, so this assembly and the kernel-per-phase assembly produce identical tokens.
// Op order of a layer: swift/Sources/QwispCore/SeedlessFusedVerify.swift:3455-3549.
#include "kernels.h"
#include "mixer_math.cuh"
#include "route.cuh"

#include <cstdio>

namespace sl {

constexpr int PS_CW = 16;                          // consumer warps
constexpr int PS_CT = PS_CW * 32;                  // consumer threads
constexpr int PS_THREADS = (PS_CW + 2) * 32;       // + static producer warp + routed-expert producer warp
constexpr int PS_SLOT = 2304;                      // bytes per ring slot: 2048 B of nibbles (or raw data) + 256 B of scales
constexpr int PS_NS = 80;                          // ring slots
constexpr long long PS_TIMEOUT = 1ll << 28;        // cycles a single wait may take (~0.14 s) before the step is abandoned
constexpr int PS_RED_UNITS = 64;
#ifndef PS_FAKE
#define PS_FAKE 0
#endif
                   // partial sums held at once: units of one phase on one SM

// ---- shared memory carve-up (bytes) ----
constexpr int PS_OFF_RING = 0;
constexpr int PS_OFF_FULL = PS_OFF_RING + PS_NS * PS_SLOT;
constexpr int PS_OFF_EMPTY = PS_OFF_FULL + PS_NS * 8;
constexpr int PS_OFF_XS = PS_OFF_EMPTY + PS_NS * 8;            // activation stage (paired order) + group sums; 12 KB
constexpr int PS_XS_BYTES = 12288;
constexpr int PS_OFF_PPLAIN = PS_OFF_XS + PS_XS_BYTES;         // normed post-attention row, plain order (router dots); 8 KB with the next
constexpr int PS_OFF_HMID = PS_OFF_PPLAIN + 4096 * 2 / 2;      // residual stream after the mixer (combine)
constexpr int PS_OFF_HRAW = PS_OFF_HMID + 4096;                // residual stream entering the layer (out-projection epilogue)
constexpr int PS_OFF_RED = PS_OFF_HRAW + 4096;                 // [units][16] partial sums
constexpr int PS_OFF_ROUTE = PS_OFF_RED + PS_RED_UNITS * 64;   // routing scratch: 544 floats + inds + scores
constexpr int PS_OFF_MISC = PS_OFF_ROUTE + 2304;               // part[16], flags, small per-phase arrays; 1536 B
constexpr int PS_SMEM_BYTES = PS_OFF_MISC + 3072;
// the mixer phases use [PS_OFF_XS, PS_OFF_HRAW) = 20 KB as scratch (the stage and the MoE rows are dead then)
constexpr int PS_MIX_BYTES = PS_OFF_HRAW - PS_OFF_XS;

struct PsMisc {                 // lives at PS_OFF_MISC
    float part[16];             // rmsnorm partial sums
    float red16[16];            // per-warp partials (gdn norms, head argmax values)
    int redi16[16];
    int abort;                  // set once a wait in this CTA ran out
    int route_layer;            // layers routed so far (written by the routing warp, read by the expert producer)
    int inds[16];
    __half scores[16];
    float gb[2][2];             // gdn: (g, beta) of the CTA's (at most two) value heads
    float v_s[32];              // gdn: conv'd v of the CTA's state rows
    float cs[32], sn[32];       // attention: rotation table
    float sm_m[8][8], sm_l[8][8];
    __align__(16) __half sk[ATT_D];   // attention: this position's key (rotated) and value
    __align__(16) __half sv[ATT_D];
    __align__(16) PLayer layer[2];    // the consumer warps' copy of the current layer's table entry (and the next one's, loaded ahead)
};
static_assert(sizeof(PsMisc) <= 3072, "misc area");
static_assert(sizeof(PLayer) % 4 == 0, "copied word by word");

// ---- the exchange protocol: 16-byte lines {d0, seq, d1, seq} ----
__device__ __forceinline__ void ll_store(uint4* line, uint32_t d0, uint32_t d1, uint32_t seq) {
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(line), "r"(d0), "r"(seq), "r"(d1), "r"(seq) : "memory");
}
// one half of a line: {d, seq} (values produced one at a time by different warps)
__device__ __forceinline__ void ll_store_half(uint2* half_line, uint32_t d, uint32_t seq) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(half_line), "r"(d), "r"(seq) : "memory");
}
// The exchange lines exist in `reps` copies `stride` lines apart; a producer writes every copy, a consumer CTA
// polls only copy (CTA index mod reps): a line polled by every CTA of the grid at once is served by its L2
// slice one request after the other, and the producers' stores queue behind the polls.
struct PsRep { size_t stride; int reps; };
__device__ __forceinline__ void ll_store_rep(uint4* line0, const PsRep& rp, uint32_t d0, uint32_t d1, uint32_t seq) {
    for (int i = 0; i < rp.reps; ++i) ll_store(line0 + (size_t)i * rp.stride, d0, d1, seq);
}
__device__ __forceinline__ void ll_store_half_rep(uint2* half0, const PsRep& rp, uint32_t d, uint32_t seq) {
    for (int i = 0; i < rp.reps; ++i) ll_store_half(half0 + (size_t)i * rp.stride * 2, d, seq);
}
struct PsWait { volatile int* s_abort; unsigned* g_abort; unsigned* err; };
__device__ __forceinline__ void ps_give_up(const PsWait& w, unsigned code) {
    *w.s_abort = 1;
    atomicOr(w.g_abort, 1u);
    atomicOr(w.err, code);
}
// A plain (relaxed, gpu scope) load of a line that another multiprocessor wrote a moment ago can be served for
// microseconds from a stale copy near the reader (measured: median 4.6 us from the store to a successful plain
// poll, 1.2 us with the read below).  So: one plain attempt for all N lines -- enough when the data has been
// there for a while -- and for every line whose flags are not in yet, a 16-byte compare-and-swap that can never
// match, which reads the line where it lives in L2 and writes nothing.
__device__ __forceinline__ void ll_read_home(const uint4* line, uint32_t& d0, uint32_t& f0, uint32_t& d1, uint32_t& f1) {
    unsigned long long lo, hi;
    asm volatile("{\n\t.reg .b128 c, n, q;\n\tmov.b128 c, {%2, %2};\n\tmov.b128 n, {%2, %2};\n\tatom.global.relaxed.gpu.cas.b128 q, [%3], c, n;\n\tmov.b128 {%0, %1}, q;\n\t}"
                 : "=l"(lo), "=l"(hi) : "l"(0xFFFFFFFFFFFFFFFFull), "l"(line) : "memory");
    d0 = (uint32_t)lo; f0 = (uint32_t)(lo >> 32); d1 = (uint32_t)hi; f1 = (uint32_t)(hi >> 32);
}
template <int N>
__device__ __forceinline__ bool ll_load_n(const uint4* const (&line)[N], uint32_t seq, uint32_t (&d)[2 * N], const PsWait& w) {
    uint32_t f0[N], f1[N];
#pragma unroll
    for (int i = 0; i < N; ++i)
        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d[2 * i]), "=r"(f0[i]), "=r"(d[2 * i + 1]), "=r"(f1[i]) : "l"(line[i]) : "memory");
    long long t0 = 0;
    for (int it = 0;; ++it) {
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i) ok = ok && (f0[i] == seq) && (f1[i] == seq);
        if (ok) return true;
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (f0[i] != seq || f1[i] != seq) ll_read_home(line[i], d[2 * i], f0[i], d[2 * i + 1], f1[i]);
        if ((it & 15) == 15) {
            if (*w.s_abort) break;
            if (t0 == 0) t0 = clock64();
            else if (clock64() - t0 > PS_TIMEOUT) { ps_give_up(w, 8u); break; }
            if ((it & 255) == 255 && *(volatile unsigned*)w.g_abort) { *w.s_abort = 1; break; }
        }
    }
#pragma unroll
    for (int i = 0; i < 2 * N; ++i) d[i] = 0;
    return false;
}
// one line
__device__ __forceinline__ bool ll_load(const uint4* line, uint32_t seq, uint32_t& d0, uint32_t& d1, const PsWait& w) {
    const uint4* const ln[1] = {line};
    uint32_t d[2];
    const bool ok = ll_load_n<1>(ln, seq, d, w);
    d0 = d[0]; d1 = d[1];
    return ok;
}
// 8 consecutive halves (two lines) as a uint4
__device__ __forceinline__ uint4 ll_load8(const uint4* lines, int first_half, uint32_t seq, const PsWait& w) {
    const uint4* const ln[2] = {lines + (first_half >> 2), lines + (first_half >> 2) + 1};
    uint32_t d[4];
    ll_load_n<2>(ln, seq, d, w);
    return make_uint4(d[0], d[1], d[2], d[3]);
}
// two runs of 8 consecutive halves, polled together
__device__ __forceinline__ void ll_load8x2(const uint4* lines_a, int first_a, const uint4* lines_b, int first_b, uint32_t seq, const PsWait& w, uint4& va, uint4& vb) {
    const uint4* const ln[4] = {lines_a + (first_a >> 2), lines_a + (first_a >> 2) + 1, lines_b + (first_b >> 2), lines_b + (first_b >> 2) + 1};
    uint32_t d[8];
    ll_load_n<4>(ln, seq, d, w);
    va = make_uint4(d[0], d[1], d[2], d[3]); vb = make_uint4(d[4], d[5], d[6], d[7]);
}
__device__ __forceinline__ __half ll_load_half(const uint4* lines, int idx, uint32_t seq, const PsWait& w) {
    uint32_t d0, d1;
    ll_load(lines + (idx >> 2), seq, d0, d1, w);
    const uint32_t d = (idx & 2) ? d1 : d0;
    return __ushort_as_half((unsigned short)((idx & 1) ? (d >> 16) : (d & 0xffffu)));
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) { return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16); }

// ---- ring ----
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
struct PsRing {
    unsigned char* slots; uint64_t* full; uint64_t* empty;
    __device__ __forceinline__ unsigned char* slot(uint32_t pos) const { return slots + (size_t)(pos % PS_NS) * PS_SLOT; }
};
// try_wait that lets the hardware park the warp (up to `ns` nanoseconds) instead of spinning: a spinning warp
// takes issue slots from the warps of its scheduler that have work (the routing warp, the producers)
__device__ __forceinline__ bool mbar_try_wait_park(uint64_t* b, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// consumer: wait until the copy into position `pos` has landed
__device__ __forceinline__ bool ring_wait(const PsRing& r, uint32_t pos, const PsWait& w) {
    uint64_t* b = r.full + (pos % PS_NS);
    const uint32_t parity = (pos / PS_NS) & 1;
    if (mbar_try_wait(b, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait_park(b, parity, 20000u)) return true;
        if (*w.s_abort) return false;
        if (clock64() - t0 > PS_TIMEOUT) { ps_give_up(w, 16u); return false; }
    }
}
// consumer: the whole warp is done reading position `pos`
__device__ __forceinline__ void ring_release(const PsRing& r, uint32_t pos, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(r.empty + (pos % PS_NS));
}
// producer warp: positions base .. base+n-1, one per lane per round; desc(i) gives the (at most two) copies
// of piece i.  A lane issues as soon as ITS slot is free; nobody waits for a neighbour.
template <typename Desc>
__device__ __forceinline__ void ring_issue(const PsRing& r, uint32_t base, int n, int lane, const PsWait& w, Desc desc) {
    for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        bool done = i >= n;
        const uint32_t pos = base + (uint32_t)i, sl = pos % PS_NS, use = pos / PS_NS;
        long long t0 = 0;
        for (int it = 0;; ++it) {
            if (!done && (use == 0 || mbar_test_wait(r.empty + sl, (use - 1) & 1))) {
                const void* s0; const void* s1; uint32_t b0, b1;
                desc(PS_FAKE ? 0 : i, s0, b0, s1, b1);
                unsigned char* dst = r.slots + (size_t)sl * PS_SLOT;
                mbar_expect_tx(r.full + sl, b0 + b1);
                bulk_g2s(dst, s0, b0, r.full + sl);
                if (b1) bulk_g2s(dst + 2048, s1, b1, r.full + sl);
                done = true;
            }
            if (__all_sync(0xffffffffu, done)) break;
            __nanosleep(60);
            if ((it & 7) == 7) {
                if (*w.s_abort) return;
                if (t0 == 0) t0 = clock64();
                else if (clock64() - t0 > PS_TIMEOUT) { ps_give_up(w, 32u); return; }
            }
        }
    }
}
__device__ __forceinline__ uint32_t ps_now() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return (uint32_t)t;
}
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(PS_CT) : "memory"); }

// ---- schedule: how many ring positions each phase of a layer takes on SM `c` (the same arithmetic in every warp) ----
__device__ __forceinline__ void ps_range(int total, int parts, int idx, int& a, int& b) {
    a = (int)((long long)total * idx / parts); b = (int)((long long)total * (idx + 1) / parts);
}
struct PsCounts { int n_in, n_state, n_out, n_router, n_gu, n_down_r, n_down_s; int gu_slot; };
__device__ __forceinline__ PsCounts ps_counts(const PsGeom& g, bool is_attn, int c) {
    PsCounts k;
    int a, b;
    const int in_N = is_attn ? g.attn_in : g.gdn_in;
    ps_range(in_N / 16, g.G, c, a, b); k.n_in = (b - a) * g.S_h;
    if (is_attn) k.n_state = 0;
    else {
        const int total = g.Hv * GDN_DV, r0 = c * g.rows_per_sm, r1 = min(total, r0 + g.rows_per_sm);
        k.n_state = r1 > r0 ? (r1 - r0) / 4 : 0;
    }
    const int outK = is_attn ? g.attn_out : g.valDim;
    ps_range(g.H / 16, g.G, c, a, b); k.n_out = (b - a) * (outK >> 8);
    k.n_router = 0;
    for (int j = c; j <= g.E; j += g.G) k.n_router += g.router_spr;
    k.gu_slot = c / g.gu_spp;
    if (k.gu_slot > g.topk) { k.gu_slot = -1; k.n_gu = 0; }
    else { ps_range(g.I / 8, g.gu_spp, c % g.gu_spp, a, b); k.n_gu = (b - a) * g.S_h; }
    ps_range(g.H / 16, g.G, c, a, b);
    k.n_down_r = (b - a) * g.topk * g.S_i; k.n_down_s = (b - a) * g.S_i;
    return k;
}
__device__ __forceinline__ uint32_t ps_layer_total(const PsCounts& k) {
    return (uint32_t)(k.n_in + k.n_state + k.n_out + k.n_router + k.n_gu + k.n_down_r + k.n_down_s);
}

// ---- one unit (16 weight rows x 256 inputs, one activation row) from a ring slot ----
// (the slot is handed back as soon as its contents are in registers)
__device__ __forceinline__ void ps_unit(const PsRing& ring, uint32_t pos, const PsWait& w, const XRegs& xr, float* red16 /*[16]*/, int lane) {
    ring_wait(ring, pos, w);
    const unsigned char* slot = ring.slot(pos);
    SliceRegs rg;
    load_slice_smem(rg, reinterpret_cast<const uint4*>(slot), reinterpret_cast<const uint4*>(slot + 2048), lane);
    ring_release(ring, pos, lane);
    float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
    compute_slice_x(rg, xr, accS, accB);
    finish_acc4(accS, accB, lane & 3, v);
    if ((lane & 3) == 0) { red16[lane >> 2] = v[0]; red16[8 + (lane >> 2)] = v[2]; }      // column 0 = the one activation row
}
// sum of a tile row's slice partials in ascending slice order (the order every GEMV kernel uses)
__device__ __forceinline__ float ps_tile_sum(const float* red, int tile_local, int slices, int row) {
    float acc = 0.f;
    for (int s = 0; s < slices; ++s) acc += red[(tile_local * slices + s) * 16 + row];
    return acc;
}

struct PsSm {
    PsRing ring;
    XStage st;                  // activation stage
    __half* pplain; __half* hmid; __half* hraw;
    float* red; float* rbuf; PsMisc* misc;
    unsigned char* mix;         // 20 KB of mixer scratch (aliases the stage and the MoE rows)
};

// RMSNorm prologue from 8-value registers: v holds this lane's values of chunk `warp` (warps < K/256)
// and wv the norm weights of the same 8 positions (fetched by the caller BEFORE it polls for v)
__device__ __forceinline__ void ps_stage_rmsnorm(const PsSm& sm, uint4 v, uint4 wv, float eps, int K, int warp, int lane, __half* plain_out) {
    const int chunks = K >> 8;
    const bool active = warp < chunks;
    if (active) {
        float ss = warp_sum(sumsq8(v));
        if (lane == 0) sm.misc->part[warp] = ss;
    }
    cbar();
    if (active) {
        const int k0 = (warp << 8) + lane * 8;
        float tot = 0.f;
        for (int c = 0; c < chunks; ++c) tot += sm.misc->part[c];
        const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), eps));
        const uint4 o = rms_apply8(v, wv, inv);
        if (plain_out) *reinterpret_cast<uint4*>(plain_out + k0) = o;
        store_staged(sm.st, 0, k0, o, lane);
    }
}

// =============================================================================================
// the kernel
// =============================================================================================
__global__ void __launch_bounds__(PS_THREADS, 1) k_step_persistent(PStepArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x;
    PsSm sm;
    sm.ring.slots = smem + PS_OFF_RING;
    sm.ring.full = reinterpret_cast<uint64_t*>(smem + PS_OFF_FULL);
    sm.ring.empty = reinterpret_cast<uint64_t*>(smem + PS_OFF_EMPTY);
    sm.st.xs = reinterpret_cast<__half*>(smem + PS_OFF_XS);
    sm.st.sxs = reinterpret_cast<float*>(smem + PS_OFF_XS + (4096 + 8) * 2);
    sm.st.part = nullptr; sm.st.stride = 4096 + 8;
    sm.pplain = reinterpret_cast<__half*>(smem + PS_OFF_PPLAIN);
    sm.hmid = reinterpret_cast<__half*>(smem + PS_OFF_HMID);
    sm.hraw = reinterpret_cast<__half*>(smem + PS_OFF_HRAW);
    sm.red = reinterpret_cast<float*>(smem + PS_OFF_RED);
    sm.rbuf = reinterpret_cast<float*>(smem + PS_OFF_ROUTE);
    sm.misc = reinterpret_cast<PsMisc*>(smem + PS_OFF_MISC);
    sm.mix = smem + PS_OFF_XS;
    if (tid == 0) {
        for (int i = 0; i < PS_NS; ++i) { mbar_init(sm.ring.full + i, 1); mbar_init(sm.ring.empty + i, 1); }
        mbar_fence_init();
        sm.misc->abort = 0; sm.misc->route_layer = 0;
    }
    __syncthreads();
    const PsGeom g = a.geom;
    const PsWait w{&sm.misc->abort, a.abort_flag, a.err};
    const PsRep rp{a.x_rep_stride, a.x_reps};
    const uint32_t seq = *(volatile unsigned*)a.step_seq;
    const int slot_id = a.segs[0].slot;

    // ======================================================================= static producer warp
    if (warp == PS_CW) {
        uint32_t base = 0;
        const int side = a.tab.parity[slot_id];
        const int kv_len0 = a.tab.kv_len[slot_id];
        for (int L = 0; L < a.n_layers; ++L) {
            const PLayer& P = a.layers[L];
            const PsCounts k = ps_counts(g, P.is_attn != 0, c);
            int t0, t1;
            {   // Pull into L2, well ahead of their use, the small per-layer constants (norm weights, conv taps, conv
                // history, decay parameters) and, for an attention layer, the cached keys / values of this CTA's split:
                // each would otherwise cost a full DRAM round trip on the critical path.  One range per lane.
                const void* pp = nullptr; uint32_t pb = 0;
                auto rng = [&](int idx, const void* p0_, size_t bytes) {
                    if (lane != idx) return;
                    const uintptr_t lo = (uintptr_t)p0_ & ~(uintptr_t)15, hi = ((uintptr_t)p0_ + bytes + 15) & ~(uintptr_t)15;
                    pp = (const void*)lo; pb = (uint32_t)(hi - lo);
                };
                rng(0, P.in_norm, (size_t)g.H * 2); rng(1, P.post_norm, (size_t)g.H * 2);
                if (!P.is_attn) {
                    const int total = g.Hv * GDN_DV, r0 = c * g.rows_per_sm, r1 = min(total, r0 + g.rows_per_sm);
                    if (r1 > r0) {
                        const int rep_ = g.Hv / g.Hk, hk0 = (r0 / GDN_DV) / rep_, hk1 = ((r1 - 1) / GDN_DV) / rep_;
                        const __half* hist_in = a.tab.conv_hist + (size_t)slot_id * a.tab.hist_stride_stream + (size_t)side * a.tab.hist_stride_side +
                                                (size_t)P.type_index * a.tab.hist_stride_layer;
                        rng(2, P.gdn_norm, 256); rng(3, P.A_log, (size_t)g.Hv * 4); rng(4, P.dt_bias, (size_t)g.Hv * 4);
                        rng(5, P.conv_w + (size_t)(hk0 * GDN_DK) * 4, 2048); rng(6, P.conv_w + (size_t)(g.keyDim + hk0 * GDN_DK) * 4, 2048);
                        rng(7, P.conv_w + (size_t)(hk1 * GDN_DK) * 4, 2048); rng(8, P.conv_w + (size_t)(g.keyDim + hk1 * GDN_DK) * 4, 2048);
                        rng(9, P.conv_w + (size_t)(2 * g.keyDim + r0) * 4, (size_t)(r1 - r0) * 16);
                        for (int j = 0; j < 3; ++j) {
                            rng(10 + 5 * j, hist_in + (size_t)j * g.convDim + hk0 * GDN_DK, 256); rng(11 + 5 * j, hist_in + (size_t)j * g.convDim + g.keyDim + hk0 * GDN_DK, 256);
                            rng(12 + 5 * j, hist_in + (size_t)j * g.convDim + hk1 * GDN_DK, 256); rng(13 + 5 * j, hist_in + (size_t)j * g.convDim + g.keyDim + hk1 * GDN_DK, 256);
                            rng(14 + 5 * j, hist_in + (size_t)j * g.convDim + 2 * g.keyDim + r0, (size_t)(r1 - r0) * 2);
                        }
                    }
                } else {
                    rng(2, P.q_norm, ATT_D * 2); rng(3, P.k_norm, ATT_D * 2);
                    const int N = kv_len0 + 1;
                    int chunk, used, p0, p1;
                    attn_split_range(N, a.nsplit, 0, chunk, used, p0, p1);
                    if (c < g.KV * used) {
                        const int kvh = c / used, split = c - kvh * used;
                        attn_split_range(N, a.nsplit, split, chunk, used, p0, p1);
                        const size_t page_elems = (size_t)a.n_attn_layers * 2 * g.KV * a.page_size * ATT_D;
                        for (int p = p0 + lane; p < p1 && p < kv_len0; p += 32) {
                            const int page = a.tab.page_table[(size_t)slot_id * a.tab.max_pages + p / a.page_size];
                            for (int which = 0; which < 2; ++which)
                                prefetch_l2_bulk(a.kv_pool + (size_t)page * page_elems + ((((size_t)P.type_index * 2 + which) * g.KV + kvh) * a.page_size + (p % a.page_size)) * ATT_D, ATT_D * 2);
                        }
                    }
                }
                if (pb) prefetch_l2_bulk(pp, pb);
            }
            ps_range((P.is_attn ? g.attn_in : g.gdn_in) / 16, g.G, c, t0, t1);
            {   // in-projection units: contiguous in the fragment-major layout
                const uint4* wr = P.r_in.wr + (size_t)t0 * g.S_h * 128; const uint4* sr = P.r_in.sr + (size_t)t0 * g.S_h * 16;
                ring_issue(sm.ring, base, k.n_in, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = wr + (size_t)i * 128; b0 = 2048; s1 = sr + (size_t)i * 16; b1 = 256; });
                base += k.n_in;
            }
            if (!P.is_attn) {   // this CTA's rows of the recurrent state: 4 rows (2048 B) per slot
                const float* S_in = a.tab.gdn_state + (size_t)slot_id * a.tab.state_stride_stream + (size_t)side * a.tab.state_stride_side +
                                    (size_t)P.type_index * a.tab.state_stride_layer + (size_t)c * g.rows_per_sm * GDN_DK;
                ring_issue(sm.ring, base, k.n_state, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = S_in + (size_t)i * 4 * GDN_DK; b0 = 2048; s1 = nullptr; b1 = 0; });
                base += k.n_state;
            }
            {
                ps_range(g.H / 16, g.G, c, t0, t1);
                const int S_o = (P.is_attn ? g.attn_out : g.valDim) >> 8;
                const uint4* wr = P.r_out.wr + (size_t)t0 * S_o * 128; const uint4* sr = P.r_out.sr + (size_t)t0 * S_o * 16;
                ring_issue(sm.ring, base, k.n_out, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = wr + (size_t)i * 128; b0 = 2048; s1 = sr + (size_t)i * 16; b1 = 256; });
                base += k.n_out;
            }
            {   // router rows (and the shared-gate row, job E) owned by this CTA: jobs c, c+G, ...
                const int spr = g.router_spr;
                ring_issue(sm.ring, base, k.n_router, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    const int jl = i / spr, part = i - jl * spr, j = c + jl * g.G;
                    const __half* row = (j == g.E) ? P.shared_gate : (P.router + (size_t)j * g.H);
                    s0 = row + (size_t)part * 1024; b0 = (uint32_t)min(2048, g.H * 2 - part * 2048); s1 = nullptr; b1 = 0; });
                base += k.n_router;
            }
            if (k.gu_slot == g.topk) {   // this CTA's part of the shared expert's gate/up
                int x0, x1; ps_range(g.I / 8, g.gu_spp, c % g.gu_spp, x0, x1);
                const uint4* wr = P.r_sh_gu.wr + (size_t)x0 * g.S_h * 128; const uint4* sr = P.r_sh_gu.sr + (size_t)x0 * g.S_h * 16;
                ring_issue(sm.ring, base, k.n_gu, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = wr + (size_t)i * 128; b0 = 2048; s1 = sr + (size_t)i * 16; b1 = 256; });
            }
            base += k.n_gu + k.n_down_r;      // the routed experts' positions belong to the other producer warp
            {   // shared expert's down projection, this CTA's output tiles
                ps_range(g.H / 16, g.G, c, t0, t1);
                const uint4* wr = P.r_sh_down.wr + (size_t)t0 * g.S_i * 128; const uint4* sr = P.r_sh_down.sr + (size_t)t0 * g.S_i * 16;
                ring_issue(sm.ring, base, k.n_down_s, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = wr + (size_t)i * 128; b0 = 2048; s1 = sr + (size_t)i * 16; b1 = 256; });
                base += k.n_down_s;
            }
            if (sm.misc->abort) return;
        }
        {   // lm_head: tiles t0..t1, positions ordered so that the 16 consumer warps (one tile each) advance together
            int t0, t1; ps_range(g.V / 16, g.G, c, t0, t1);
            const int ntl = t1 - t0, S = g.S_h, full = ntl / 16, rem = ntl - full * 16;
            ring_issue(sm.ring, base, ntl * S, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                int tl, s;
                if (i < full * 16 * S) { const int rd = i / (16 * S), q = i - rd * 16 * S; s = q >> 4; tl = rd * 16 + (q & 15); }
                else { const int q = i - full * 16 * S; s = q / rem; tl = full * 16 + (q - s * rem); }
                const size_t u = (size_t)(t0 + tl) * S + s;
                s0 = a.lm_head.wr + u * 128; b0 = 2048; s1 = a.lm_head.sr + u * 16; b1 = 256; });
        }
        return;
    }
    // ======================================================================= routed-expert producer warp
    if (warp == PS_CW + 1) {
        uint32_t base = 0;
        for (int L = 0; L < a.n_layers; ++L) {
            const PLayer& P = a.layers[L];
            const PsCounts k = ps_counts(g, P.is_attn != 0, c);
            const uint32_t gu_base = base + k.n_in + k.n_state + k.n_out + k.n_router;
            base += ps_layer_total(k);
            const bool has_gu = k.gu_slot >= 0 && k.gu_slot < g.topk && k.n_gu > 0;
            if (!has_gu && k.n_down_r == 0) continue;
            {   // wait for this layer's routing (written by the routing warp of this CTA)
                long long t0 = 0;
                for (int it = 0; *(volatile int*)&sm.misc->route_layer <= L; ++it) {
                    __nanosleep(32);
                    if ((it & 15) == 15) {
                        if (sm.misc->abort) return;
                        if (t0 == 0) t0 = clock64();
                        else if (clock64() - t0 > PS_TIMEOUT) { ps_give_up(w, 64u); return; }
                    }
                }
            }
            __syncwarp();
            if (has_gu) {
                const int e = *(volatile int*)&sm.misc->inds[k.gu_slot];
                int x0, x1; ps_range(g.I / 8, g.gu_spp, c % g.gu_spp, x0, x1);
                const size_t u0 = ((size_t)e * (g.I / 8) + x0) * g.S_h;
                ring_issue(sm.ring, gu_base, k.n_gu, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    s0 = P.r_gu.wr + (u0 + i) * 128; b0 = 2048; s1 = P.r_gu.sr + (u0 + i) * 16; b1 = 256; });
            }
            if (k.n_down_r) {
                int t0, t1; ps_range(g.H / 16, g.G, c, t0, t1);
                const int per_tile = g.topk * g.S_i;
                ring_issue(sm.ring, gu_base + k.n_gu, k.n_down_r, lane, w, [&](int i, const void*& s0, uint32_t& b0, const void*& s1, uint32_t& b1) {
                    const int tl = i / per_tile, q = i - tl * per_tile, kk = q / g.S_i, s = q - kk * g.S_i;
                    const int e = *(volatile int*)&sm.misc->inds[kk];
                    const size_t u = ((size_t)e * (g.H / 16) + t0 + tl) * g.S_i + s;
                    s0 = P.r_down.wr + u * 128; b0 = 2048; s1 = P.r_down.sr + u * 16; b1 = 256; });
            }
        }
        return;
    }

    // ======================================================================= consumer warps
    const int r = lane >> 2, t = lane & 3;
    const int kv_len0 = a.tab.kv_len[slot_id];
    const int side = a.tab.parity[slot_id];
    uint32_t base = 0;                                       // ring position of the current phase's first piece
    if (tid < 32) rope_table_entry(a.theta, kv_len0, tid, sm.misc->cs[tid], sm.misc->sn[tid]);   // every attention layer rotates by the same position
    int tok = a.tok_in[0];
    if (tok < 0 || tok >= g.V) tok = 0;

    // optional timeline (profiling): nanosecond stamps of this CTA's phase boundaries, [CTA][layer + 1][24]
    uint32_t* tl_cta = a.timeline ? a.timeline + (size_t)c * (a.n_layers + 1) * 24 : nullptr;
    const uint32_t t_start = 0;        // stamps are absolute (low 32 bits of the global nanosecond timer): comparable across CTAs
#define PS_MARK(L_, i_) do { if (tl_cta && tid == 0) tl_cta[(L_) * 24 + (i_)] = ps_now() - t_start; } while (0)
    {   // layer 0's table entry; every later entry is copied in during the layer before it
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.layers);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.misc->layer[0]);
        for (int i = tid; i < (int)(sizeof(PLayer) / 4); i += PS_CT) dst[i] = src[i];
        cbar();
    }
    for (int L = 0; L < a.n_layers; ++L) {
        const PLayer& P = sm.misc->layer[L & 1];
        const bool is_attn = P.is_attn != 0;
        const PsCounts k = ps_counts(g, is_attn, c);
        if (L + 1 < a.n_layers && warp == PS_CW - 2) {       // visible to all after the barriers that follow in this layer
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a.layers + L + 1);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.misc->layer[(L + 1) & 1]);
            for (int i = lane; i < (int)(sizeof(PLayer) / 4); i += 32) dst[i] = src[i];
        }
        PS_MARK(L, 0);
        if (tl_cta && tid == 0 && L == 2) {       // profiling only: round-trip time of a polled line (8 dependent loads), and of a store followed by a load of it
            uint32_t a0 = 0, f0, b0, f1;
            const uint4* ln = a.xbuf + (size_t)(c % a.x_reps) * a.x_rep_stride;
            const uint32_t t0 = ps_now();
            for (int i = 0; i < 8; ++i)
                asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(f0), "=r"(b0), "=r"(f1) : "l"(ln + (a0 & 1)) : "memory");
            tl_cta[L * 24 + 17] = ps_now() - t0 + (a0 & 1);
        }
        uint4* Xw = a.xbuf + (size_t)L * a.x_stride;                                  // this layer's exchange lines, copy 0 (stores go to every copy)
        const uint4* X = Xw + (size_t)(c % a.x_reps) * a.x_rep_stride;                // the copy this CTA reads
        uint4* Xnext = a.xbuf + (size_t)(L + 1) * a.x_stride;
        // ---------------------------------------------------------------- in-projection
        {
            const int chunks = g.S_h;
            uint4 v = make_uint4(0, 0, 0, 0), nwv = make_uint4(0, 0, 0, 0);
            if (warp < chunks) {
                const int k0 = (warp << 8) + lane * 8;
                nwv = *reinterpret_cast<const uint4*>(P.in_norm + k0);
                if (L == 0) v = __ldg(reinterpret_cast<const uint4*>(a.embed + (size_t)tok * g.H + k0));
                else v = ll_load8(X + a.x_off_h, k0, seq, w);
                *reinterpret_cast<uint4*>(sm.hraw + k0) = v;
            }
            ps_stage_rmsnorm(sm, v, nwv, a.eps, g.H, warp, lane, nullptr);
            cbar();
            PS_MARK(L, 1);
            int t0, t1; ps_range((is_attn ? g.attn_in : g.gdn_in) / 16, g.G, c, t0, t1);
            XRegs xr;
            load_xregs(xr, sm.st, warp & (g.S_h - 1), r, t, 1);
            for (int u = warp; u < k.n_in; u += PS_CW) {
                ps_unit(sm.ring, base + u, w, xr, sm.red + u * 16, lane);
            }
            cbar();
            PS_MARK(L, 2);
            const int n_out = (t1 - t0) * 16;
            for (int i0 = 0; i0 < n_out; i0 += PS_CT) {
                const int i = i0 + tid;
                __half val = f2h(0.f);
                if (i < n_out) val = f2h(ps_tile_sum(sm.red, i >> 4, g.S_h, i & 15));
                const uint32_t me = __half_as_ushort(val);
                const uint32_t h1 = __shfl_down_sync(0xffffffffu, me, 1), h2 = __shfl_down_sync(0xffffffffu, me, 2), h3 = __shfl_down_sync(0xffffffffu, me, 3);
                if (i < n_out && (i & 3) == 0) ll_store_rep(Xw + a.x_off_in + ((t0 * 16 + i) >> 2), rp, me | (h1 << 16), h2 | (h3 << 16), seq);
            }
            base += k.n_in;
        }
        PS_MARK(L, 3);
        // ---------------------------------------------------------------- mixer core
        if (!is_attn) {
            // --- gated delta net: this CTA owns state rows [r0, r1) (whole groups of 4, inside at most two value heads)
            const int total = g.Hv * GDN_DV, r0 = c * g.rows_per_sm, r1 = min(total, r0 + g.rows_per_sm);
            const int rep = g.Hv / g.Hk;
            float* q_s = reinterpret_cast<float*>(sm.mix);                 // [2 key heads][128]
            float* k_s = q_s + 256;
            if (r1 > r0) {
                const int hv0 = r0 / GDN_DV, hv1 = (r1 - 1) / GDN_DV, hk0 = hv0 / rep, hk1 = hv1 / rep;
                const __half* hist_in = a.tab.conv_hist + (size_t)slot_id * a.tab.hist_stride_stream + (size_t)side * a.tab.hist_stride_side +
                                        (size_t)P.type_index * a.tab.hist_stride_layer;
                __half* hist_out = a.tab.conv_hist + (size_t)slot_id * a.tab.hist_stride_stream + (size_t)(side ^ 1) * a.tab.hist_stride_side +
                                   (size_t)P.type_index * a.tab.hist_stride_layer;
                const uint4* XI = X + a.x_off_in;
                // step A: conv + SiLU of the q and k channels of the key heads this CTA needs (256 threads per head)
                {
                    const int j = tid >> 8, isk = (tid >> 7) & 1, cl = tid & 127;
                    const int hk = j ? hk1 : hk0;
                    const bool need = (j == 0) || (hk1 != hk0);
                    float qc = 0.f;
                    if (need) {
                        const int ch = (isk ? g.keyDim : 0) + hk * GDN_DK + cl;
                        const float4 cw = *reinterpret_cast<const float4*>(P.conv_w + (size_t)ch * 4);
                        const __half h0 = hist_in[ch], h1 = hist_in[(size_t)g.convDim + ch], h2 = hist_in[(size_t)2 * g.convDim + ch];
                        const __half x = ll_load_half(XI, ch, seq, w);
                        qc = gdn_conv_silu(h2f(h0), h2f(h1), h2f(h2), h2f(x), cw);
                        // the key head's q / k history is written by the CTA that holds the head's first state row
                        const int first_row = hk * rep * GDN_DV;
                        if (first_row >= r0 && first_row < r1) {
                            hist_out[ch] = h1; hist_out[(size_t)g.convDim + ch] = h2; hist_out[(size_t)2 * g.convDim + ch] = x;
                        }
                    }
                    // v channels of this CTA's rows, decay / beta of its value heads
                    if (tid < r1 - r0) {
                        const int ch = 2 * g.keyDim + r0 + tid;
                        const float4 cw = *reinterpret_cast<const float4*>(P.conv_w + (size_t)ch * 4);
                        const __half h0 = hist_in[ch], h1 = hist_in[(size_t)g.convDim + ch], h2 = hist_in[(size_t)2 * g.convDim + ch];
                        const __half x = ll_load_half(XI, ch, seq, w);
                        sm.misc->v_s[tid] = gdn_conv_silu(h2f(h0), h2f(h1), h2f(h2), h2f(x), cw);
                        hist_out[ch] = h1; hist_out[(size_t)g.convDim + ch] = h2; hist_out[(size_t)2 * g.convDim + ch] = x;
                    }
                    if (tid >= 64 && tid < 66) {
                        const int hv = (tid == 64) ? hv0 : hv1;
                        const __half bh = ll_load_half(XI, g.convDim + g.valDim + hv, seq, w);
                        const __half ah = ll_load_half(XI, g.convDim + g.valDim + g.Hv + hv, seq, w);
                        gdn_gate(bh, ah, P.A_log[hv], P.dt_bias[hv], sm.misc->gb[tid - 64][0], sm.misc->gb[tid - 64][1]);
                    }
                    const float ss = warp_sum(qc * qc);
                    if (lane == 0) sm.misc->red16[warp] = ss;
                    cbar();
                    if (need) {
                        const int w0 = (tid >> 7) * 4;
                        const float inv = gdn_head_inv(sm.misc->red16[w0], sm.misc->red16[w0 + 1], sm.misc->red16[w0 + 2], sm.misc->red16[w0 + 3], a.eps);
                        if (isk) k_s[j * 128 + cl] = gdn_scale_k(qc, inv);
                        else q_s[j * 128 + cl] = gdn_scale_q(qc, inv);
                    }
                    cbar();
                }
                // step B: the state rows, four per ring slot, one slot per warp at a time
                float* S_out = a.tab.gdn_state + (size_t)slot_id * a.tab.state_stride_stream + (size_t)(side ^ 1) * a.tab.state_stride_side +
                               (size_t)P.type_index * a.tab.state_stride_layer;
                for (int q = warp; q < k.n_state; q += PS_CW) {
                    const int row0 = r0 + 4 * q, hv = row0 / GDN_DV, jh = (hv == hv0) ? 0 : 1, jk = (hv / rep == hk0) ? 0 : 1;
                    const float4 kq = *reinterpret_cast<const float4*>(k_s + jk * 128 + lane * 4);
                    const float4 qq = *reinterpret_cast<const float4*>(q_s + jk * 128 + lane * 4);
                    const float gg = sm.misc->gb[jh][0], beta = sm.misc->gb[jh][1];
                    ring_wait(sm.ring, base + q, w);
                    const float4* rows = reinterpret_cast<const float4*>(sm.ring.slot(base + q));
                    float4 S[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) S[i] = rows[i * 32 + lane];
                    ring_release(sm.ring, base + q, lane);
                    __half o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        o[i] = f2h(gdn_row_step(S[i], gg, kq, qq, sm.misc->v_s[4 * q + i], beta));
                        *reinterpret_cast<float4*>(S_out + (size_t)(row0 + i) * GDN_DK + lane * 4) = S[i];
                    }
                    if (lane == 0) ll_store_rep(Xw + a.x_off_mix + (row0 >> 2), rp, pack_h2(o[0], o[1]), pack_h2(o[2], o[3]), seq);
                }
            }
            base += k.n_state;
            cbar();                                                        // the scratch is the stage of the next phase
        } else {
            // --- full attention: (split, kv head) work items, then one warp per head merges the splits
            const int pos = kv_len0, N = pos + 1;
            int chunk, used, p0, p1;
            attn_split_range(N, a.nsplit, 0, chunk, used, p0, p1);
            const uint4* XI = X + a.x_off_in;
            uint4* XP = a.xatt + (size_t)P.type_index * a.xatt_stride;     // partial lines: [head][split][129]
            __half* sq = reinterpret_cast<__half*>(sm.mix);                // [8][256]
            __half* sk = sm.misc->sk; __half* sv = sm.misc->sv;
            float* mbuf = reinterpret_cast<float*>(sm.mix + 8 * ATT_D * 2);               // [8 key warps][2 heads][256] = 16 KB
            const size_t page_elems = (size_t)a.n_attn_layers * 2 * g.KV * a.page_size * ATT_D;
            auto kvp = [&](int p, int which, int kvh) -> __half* {
                const int page = a.tab.page_table[(size_t)slot_id * a.tab.max_pages + p / a.page_size];
                return a.kv_pool + (size_t)page * page_elems + ((((size_t)P.type_index * 2 + which) * g.KV + kvh) * a.page_size + (p % a.page_size)) * ATT_D;
            };
            for (int wi = c; wi < g.KV * used; wi += g.G) {
                const int kvh = wi / used, split = wi - kvh * used;
                attn_split_range(N, a.nsplit, split, chunk, used, p0, p1);
                const bool own = pos >= p0 && pos < p1;
                if (warp < ATT_G) {
                    const uint4 v = ll_load8(XI, (kvh * ATT_G + warp) * 2 * ATT_D + lane * 8, seq, w);
                    reinterpret_cast<uint4*>(sq + warp * ATT_D)[lane] = norm_rope_head_tab(v, P.q_norm, a.eps, sm.misc->cs, sm.misc->sn, lane);
                } else if (own && warp == ATT_G) {
                    const uint4 v = ll_load8(XI, g.NH * 2 * ATT_D + kvh * ATT_D + lane * 8, seq, w);
                    const uint4 ko = norm_rope_head_tab(v, P.k_norm, a.eps, sm.misc->cs, sm.misc->sn, lane);
                    reinterpret_cast<uint4*>(sk)[lane] = ko;
                    reinterpret_cast<uint4*>(kvp(pos, 0, kvh))[lane] = ko;
                } else if (own && warp == ATT_G + 1) {
                    const uint4 vo = ll_load8(XI, g.NH * 2 * ATT_D + g.KV * ATT_D + kvh * ATT_D + lane * 8, seq, w);
                    reinterpret_cast<uint4*>(sv)[lane] = vo;
                    reinterpret_cast<uint4*>(kvp(pos, 1, kvh))[lane] = vo;
                }
                cbar();
                const int kw = warp & 7;
                for (int pass = 0; pass < 2; ++pass) {
                    const int hp = (warp >> 3) + 2 * pass;                // this warp's pair of heads: 2hp, 2hp+1 (of the kv head's 8)
                    float q[2][8], mx[2], l[2], acc[2][8];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint4 qv = reinterpret_cast<const uint4*>(sq + (2 * hp + hh) * ATT_D)[lane];
                        const __half* qh = reinterpret_cast<const __half*>(&qv);
                        mx[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) { q[hh][i] = 0.0625f * h2f(qh[i]); acc[hh][i] = 0.f; }
                    }
                    auto load_kv = [&](int p, uint4& kk, uint4& vv) {
                        if (own && p == pos) { kk = reinterpret_cast<const uint4*>(sk)[lane]; vv = reinterpret_cast<const uint4*>(sv)[lane]; }
                        else { kk = reinterpret_cast<const uint4*>(kvp(p, 0, kvh))[lane]; vv = reinterpret_cast<const uint4*>(kvp(p, 1, kvh))[lane]; }
                    };
                    uint4 kcur = make_uint4(0, 0, 0, 0), vcur = make_uint4(0, 0, 0, 0);
                    if (p0 + kw < p1) load_kv(p0 + kw, kcur, vcur);
                    for (int p = p0 + kw; p < p1; p += 8) {
                        uint4 knext = make_uint4(0, 0, 0, 0), vnext = make_uint4(0, 0, 0, 0);
                        if (p + 8 < p1) load_kv(p + 8, knext, vnext);
                        const __half* kh = reinterpret_cast<const __half*>(&kcur);
                        const __half* vh = reinterpret_cast<const __half*>(&vcur);
                        float kf[8], vf[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) { kf[i] = h2f(kh[i]); vf[i] = h2f(vh[i]); }
                        attn_key_step(q[0], kf, vf, mx[0], l[0], acc[0]);
                        attn_key_step(q[1], kf, vf, mx[1], l[1], acc[1]);
                        kcur = knext; vcur = vnext;
                    }
                    if (lane == 0) {
                        sm.misc->sm_m[kw][2 * hp] = mx[0]; sm.misc->sm_l[kw][2 * hp] = l[0];
                        sm.misc->sm_m[kw][2 * hp + 1] = mx[1]; sm.misc->sm_l[kw][2 * hp + 1] = l[1];
                    }
                    cbar();
                    // the four heads of this pass are 4*pass .. 4*pass+3 (warps 0-7 hold 4p, 4p+1; warps 8-15 hold 4p+2, 4p+3)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int head = 2 * hp + hh;                      // within the kv head
                        float m8[8];
#pragma unroll
                        for (int x = 0; x < 8; ++x) m8[x] = sm.misc->sm_m[x][head];
                        const float gm = attn_warps_max(m8);
                        const float f = (mx[hh] == -INFINITY) ? 0.f : __expf(mx[hh] - gm);
                        float4* dst = reinterpret_cast<float4*>(mbuf + ((size_t)kw * 2 + (warp >> 3)) * ATT_D + lane * 8);
                        dst[0] = make_float4(acc[hh][0] * f, acc[hh][1] * f, acc[hh][2] * f, acc[hh][3] * f);
                        dst[1] = make_float4(acc[hh][4] * f, acc[hh][5] * f, acc[hh][6] * f, acc[hh][7] * f);
                        cbar();
                        {   // 512 threads: (which of the two heads in the buffer, dim)
                            const int which = tid >> 8, d = tid & 255;
                            const int hd = kvh * ATT_G + 4 * pass + 2 * which + hh;      // global head index
                            float o = 0.f;
#pragma unroll
                            for (int x = 0; x < 8; ++x) o += mbuf[((size_t)x * 2 + which) * ATT_D + d];
                            const uint32_t me = __float_as_uint(o), nb = __shfl_down_sync(0xffffffffu, me, 1);
                            uint4* dstl = XP + ((size_t)hd * a.nsplit + split) * 129;
                            if ((d & 1) == 0) ll_store(dstl + (d >> 1), me, nb, seq);
                            if (d == 0) {
                                float mm[8], ll8[8];
                                const int hl = 4 * pass + 2 * which + hh;
                                for (int x = 0; x < 8; ++x) { mm[x] = sm.misc->sm_m[x][hl]; ll8[x] = sm.misc->sm_l[x][hl]; }
                                const float gm2 = attn_warps_max(mm);
                                const float ls = attn_warps_lsum(mm, ll8, gm2);
                                ll_store(dstl + 128, __float_as_uint(gm2), __float_as_uint(ls), seq);
                            }
                        }
                        cbar();
                    }
                }
            }
            // merge of the splits: head hd by warp 0 of CTA G-1-hd (the work items sit on the low CTAs)
            for (int hd = g.G - 1 - c; hd < g.NH; hd += g.G) {
                if (hd < 0) break;
                if (warp == 0) {
                    const uint4 gvv = ll_load8(XI, hd * 2 * ATT_D + ATT_D + lane * 8, seq, w);
                    const uint4* src = XP + (size_t)hd * a.nsplit * 129;
                    const uint4 outv = attn_merge_splits(used, lane, gvv,
                        [&](int sp, float4& x0, float4& x1) {
                            uint32_t d[8];
                            const uint4* l0 = src + (size_t)sp * 129 + lane * 4;
                            const uint4* const ln[4] = {l0, l0 + 1, l0 + 2, l0 + 3};
                            ll_load_n<4>(ln, seq, d, w);
                            x0 = make_float4(__uint_as_float(d[0]), __uint_as_float(d[1]), __uint_as_float(d[2]), __uint_as_float(d[3]));
                            x1 = make_float4(__uint_as_float(d[4]), __uint_as_float(d[5]), __uint_as_float(d[6]), __uint_as_float(d[7])); },
                        [&](int sp) { uint32_t d0, d1; ll_load(src + (size_t)sp * 129 + 128, seq, d0, d1, w); return make_float2(__uint_as_float(d0), __uint_as_float(d1)); });
                    uint4* dst = Xw + a.x_off_mix + ((hd * ATT_D + lane * 8) >> 2);
                    ll_store_rep(dst, rp, outv.x, outv.y, seq);
                    ll_store_rep(dst + 1, rp, outv.z, outv.w, seq);
                }
            }
            cbar();
        }
        PS_MARK(L, 4);
        // ---------------------------------------------------------------- out-projection (+ residual)
        {
            int t0, t1; ps_range(g.H / 16, g.G, c, t0, t1);
            const int outK = is_attn ? g.attn_out : g.valDim, S_o = outK >> 8;
            if (t1 > t0) {
                for (int ch = warp; ch < S_o; ch += PS_CW) {
                    const int k0 = (ch << 8) + lane * 8;
                    uint4 v, o;
                    if (is_attn) { v = ll_load8(X + a.x_off_mix, k0, seq, w); o = v; }
                    else {
                        const uint4 wv = *reinterpret_cast<const uint4*>(P.gdn_norm + (k0 & 127));
                        uint4 zv;
                        ll_load8x2(X + a.x_off_mix, k0, X + a.x_off_in, g.convDim + k0, seq, w, v, zv);
                        o = P.gdn_norm32 ? normgate8<PRO_NORMGATE32>(v, zv, wv, P.gdn_norm32, k0, a.eps) : normgate8<PRO_NORMGATE>(v, zv, wv, nullptr, k0, a.eps);
                    }
                    store_staged(sm.st, 0, k0, o, lane);
                }
                cbar();
                PS_MARK(L, 5);
                XRegs xr;
                load_xregs(xr, sm.st, warp & (S_o - 1), r, t, 1);
                for (int u = warp; u < k.n_out; u += PS_CW) {
                    ps_unit(sm.ring, base + u, w, xr, sm.red + u * 16, lane);
                }
                cbar();
                const int n_out = (t1 - t0) * 16;
                for (int i0 = 0; i0 < n_out; i0 += PS_CT) {
                    const int i = i0 + tid;
                    __half val = f2h(0.f);
                    if (i < n_out) val = hadd_rn(sm.hraw[t0 * 16 + i], f2h(ps_tile_sum(sm.red, i >> 4, S_o, i & 15)));
                    const uint32_t me = __half_as_ushort(val);
                    const uint32_t h1 = __shfl_down_sync(0xffffffffu, me, 1), h2 = __shfl_down_sync(0xffffffffu, me, 2), h3 = __shfl_down_sync(0xffffffffu, me, 3);
                    if (i < n_out && (i & 3) == 0) ll_store_rep(Xw + a.x_off_hm + ((t0 * 16 + i) >> 2), rp, me | (h1 << 16), h2 | (h3 << 16), seq);
                }
            }
            base += k.n_out;
        }
        PS_MARK(L, 6);
        // ---------------------------------------------------------------- post-attention norm, router logits, shared gate logit
        {
            uint4 v = make_uint4(0, 0, 0, 0), nwv = make_uint4(0, 0, 0, 0);
            if (warp < g.S_h) {
                const int k0 = (warp << 8) + lane * 8;
                nwv = *reinterpret_cast<const uint4*>(P.post_norm + k0);
                v = ll_load8(X + a.x_off_hm, k0, seq, w);
                *reinterpret_cast<uint4*>(sm.hmid + k0) = v;
            }
            ps_stage_rmsnorm(sm, v, nwv, a.eps, g.H, warp, lane, sm.pplain);
            cbar();
            PS_MARK(L, 7);
            const int spr = g.router_spr, njobs = k.n_router / spr;
            for (int jl = 0; jl < njobs; ++jl) {
                if (warp != ((8 + jl) & 15)) continue;
                const int j = c + jl * g.G;
                float acc = 0.f;
                for (int part = 0; part < spr; ++part) {
                    const uint32_t pz = base + jl * spr + part;
                    ring_wait(sm.ring, pz, w);
                    const __half* wrow = reinterpret_cast<const __half*>(sm.ring.slot(pz));
                    const int nb = min(4, (g.H >> 8) - part * 4);      // 256-wide blocks in this slot
                    for (int kb = 0; kb < nb; ++kb) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(wrow + kb * 256 + lane * 8);
                        const uint4 xv = *reinterpret_cast<const uint4*>(sm.pplain + (part * 4 + kb) * 256 + lane * 8);
                        const __half* wh = reinterpret_cast<const __half*>(&wv);
                        const __half* xh = reinterpret_cast<const __half*>(&xv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc = fmaf(h2f(xh[i]), h2f(wh[i]), acc);
                    }
                    ring_release(sm.ring, pz, lane);
                }
                const float d = warp_sum(acc);
                if (tl_cta && lane == 0 && jl == 0) tl_cta[L * 24 + 16] = ps_now() - t_start;
                if (lane == 0) {
                    const uint32_t bits = (uint32_t)__half_as_ushort(f2h(d));
                    if (j == g.E) ll_store_rep(Xw + a.x_off_lg + (j >> 1), rp, bits, 0u, seq);      // the shared-gate logit has its line to itself (E is even)
                    else ll_store_half_rep(reinterpret_cast<uint2*>(Xw + a.x_off_lg) + j, rp, bits, seq);
                }
            }
            base += k.n_router;
        }
        PS_MARK(L, 8);
        // ---------------------------------------------------------------- routing, gate/up of this CTA's expert slot
        {
            const bool in_moe = (k.gu_slot >= 0 && k.n_gu > 0) || k.n_down_s > 0;
            if (in_moe && warp == PS_CW - 1) {
                // every CTA routes the row itself from the logits (deterministic, so all agree)
                __half* lrow = reinterpret_cast<__half*>(sm.rbuf + 256);          // E <= 256 halves behind the 256 floats the routing itself uses
                {   // lane l takes logits 8l .. 8l+7 (four lines), polled together
                    const int e0 = lane * 8;
                    if (e0 < g.E) {
                        const uint4* base_l = X + a.x_off_lg + (e0 >> 1);
                        const uint4* const ln[4] = {base_l, base_l + 1, base_l + 2, base_l + 3};
                        uint32_t d[8];
                        ll_load_n<4>(ln, seq, d, w);
#pragma unroll
                        for (int i = 0; i < 8; ++i) lrow[e0 + i] = __ushort_as_half((unsigned short)d[i]);
                    }
                }
                __syncwarp();
                if (tl_cta && lane == 0) tl_cta[L * 24 + 15] = ps_now() - t_start;
                // the chosen experts are published (route_layer = L + 1) as soon as they are known: the producer warp starts the
                // weight copies while this warp goes on with the gates
                route_row_smem(lrow, g.E, g.topk, sm.misc->inds, sm.misc->scores, sm.rbuf, lane, &sm.misc->route_layer, L + 1);
                if (lane == 0 && tl_cta) tl_cta[L * 24 + 9] = ps_now() - t_start;
            }
            if (k.gu_slot >= 0 && k.n_gu > 0) {
                int x0, x1; ps_range(g.I / 8, g.gu_spp, c % g.gu_spp, x0, x1);
                XRegs xr;
                load_xregs(xr, sm.st, warp & (g.S_h - 1), r, t, 1);        // the staged normed row
                for (int u = warp; u < k.n_gu; u += PS_CW) {
                    ps_unit(sm.ring, base + u, w, xr, sm.red + u * 16, lane);
                }
                cbar();
                PS_MARK(L, 10);
                const int n_out = (x1 - x0) * 8;                            // SwiGLU outputs of this CTA
                for (int i0 = 0; i0 < n_out; i0 += PS_CT) {
                    const int i = i0 + tid;
                    __half val = f2h(0.f);
                    if (i < n_out) {
                        const __half gq = f2h(ps_tile_sum(sm.red, i >> 3, g.S_h, i & 7)), uq = f2h(ps_tile_sum(sm.red, i >> 3, g.S_h, (i & 7) + 8));
                        val = swiglu_h(gq, uq);
                    }
                    const uint32_t me = __half_as_ushort(val);
                    const uint32_t h1 = __shfl_down_sync(0xffffffffu, me, 1), h2 = __shfl_down_sync(0xffffffffu, me, 2), h3 = __shfl_down_sync(0xffffffffu, me, 3);
                    if (i < n_out && (i & 3) == 0) ll_store_rep(Xw + a.x_off_hb + ((k.gu_slot * g.I + x0 * 8 + i) >> 2), rp, me | (h1 << 16), h2 | (h3 << 16), seq);
                }
            }
            base += k.n_gu;
        }
        PS_MARK(L, 11);
        // ---------------------------------------------------------------- down projections of this CTA's output tiles + combine
        {
            int t0, t1; ps_range(g.H / 16, g.G, c, t0, t1);
            const int nsl = g.topk + 1, ntl = t1 - t0;
            cbar();                                                   // gate/up readers of the stage are done; routing results visible
            if (ntl > 0) {
                // stage the SwiGLU rows of all slots: [slot][I + 8] halves, group sums [slot][I/64][8]
                __half* xs2 = sm.st.xs;
                float* sxs2 = reinterpret_cast<float*>(sm.st.xs + (size_t)nsl * (g.I + 8));
                const int chunks = g.I >> 8;
                for (int u = warp; u < nsl * chunks; u += PS_CW) {
                    const int sidx = u / chunks, ch = u - sidx * chunks, k0 = ch * 256 + lane * 8;
                    XStage ss; ss.xs = xs2 + (size_t)sidx * (g.I + 8); ss.sxs = sxs2 + (size_t)sidx * (g.I >> 6) * 8; ss.part = nullptr; ss.stride = g.I + 8;
                    const uint4 v = ll_load8(X + a.x_off_hb, sidx * g.I + k0, seq, w);
                    store_staged(ss, 0, k0, v, lane);
                }
                cbar();
                PS_MARK(L, 12);
                const int nunits = ntl * nsl * g.S_i;
                for (int u = warp; u < nunits; u += PS_CW) {
                    const int tl = u / (nsl * g.S_i), q = u - tl * nsl * g.S_i, kk = q / g.S_i, s = q - kk * g.S_i;
                    const uint32_t pz = (kk < g.topk) ? base + (uint32_t)((tl * g.topk + kk) * g.S_i + s) : base + (uint32_t)k.n_down_r + (uint32_t)(tl * g.S_i + s);
                    XStage ss; ss.xs = xs2 + (size_t)kk * (g.I + 8); ss.sxs = sxs2 + (size_t)kk * (g.I >> 6) * 8; ss.part = nullptr; ss.stride = g.I + 8;
                    XRegs xr;
                    load_xregs(xr, ss, s, r, t, 1);
                    ps_unit(sm.ring, pz, w, xr, sm.red + u * 16, lane);
                }
                cbar();
                PS_MARK(L, 13);
                // fp16 weighted sum in ascending k (SeedlessFusedVerify.swift:462-471), + sigmoid(gate logit) * shared
                // (:474-484), + residual (SeedlessMetalForward.swift:1024-1028); each slot's value is rounded to fp16 first
                const int n_out = ntl * 16;
                for (int i0 = 0; i0 < n_out; i0 += PS_CT) {
                    const int i = i0 + tid;
                    __half val = f2h(0.f);
                    if (i < n_out) {
                        const int tl = i >> 4, row = i & 15;
                        __half acc = f2h(0.0f);
                        for (int kk = 0; kk < g.topk; ++kk)
                            acc = hadd_rn(acc, hmul_rn(f2h(ps_tile_sum(sm.red, tl * nsl + kk, g.S_i, row)), sm.misc->scores[kk]));
                        const __half sgl = ll_load_half(X + a.x_off_lg, 2 * g.E, seq, w);      // job E sits in half-line E: halves index 2E
                        const __half res = hadd_rn(acc, hmul_rn(sigmoid_h(sgl), f2h(ps_tile_sum(sm.red, tl * nsl + g.topk, g.S_i, row))));
                        val = hadd_rn(sm.hmid[t0 * 16 + i], res);
                    }
                    const uint32_t me = __half_as_ushort(val);
                    const uint32_t h1 = __shfl_down_sync(0xffffffffu, me, 1), h2 = __shfl_down_sync(0xffffffffu, me, 2), h3 = __shfl_down_sync(0xffffffffu, me, 3);
                    if (i < n_out && (i & 3) == 0) ll_store_rep(Xnext + a.x_off_h + ((t0 * 16 + i) >> 2), rp, me | (h1 << 16), h2 | (h3 << 16), seq);
                }
            }
            base += k.n_down_r + k.n_down_s;
            cbar();
            PS_MARK(L, 14);
        }
    }
    // ======================================================================= final norm, lm_head, argmax
    {
        uint4* Xw = a.xbuf + (size_t)a.n_layers * a.x_stride;
        const uint4* X = Xw + (size_t)(c % a.x_reps) * a.x_rep_stride;
        uint4 v = make_uint4(0, 0, 0, 0), nwv = make_uint4(0, 0, 0, 0);
        if (warp < g.S_h) {
            nwv = *reinterpret_cast<const uint4*>(a.final_norm + (warp << 8) + lane * 8);
            v = ll_load8(X + a.x_off_h, (warp << 8) + lane * 8, seq, w);
        }
        PS_MARK(a.n_layers, 0);
        ps_stage_rmsnorm(sm, v, nwv, a.eps, g.H, warp, lane, nullptr);
        cbar();
        PS_MARK(a.n_layers, 1);
        int t0, t1; ps_range(g.V / 16, g.G, c, t0, t1);
        const int ntl = t1 - t0, S = g.S_h, full = ntl / 16, rem = ntl - full * 16;
        float best[2] = {-INFINITY, -INFINITY}; int besti[2] = {0x7fffffff, 0x7fffffff};
        for (int rd = 0; rd * 16 + warp < ntl; ++rd) {
            const int tl = rd * 16 + warp;
            const int width = (rd < full) ? 16 : rem;
            float tot0 = 0.f, tot2 = 0.f;
            for (int s = 0; s < S; ++s) {
                const uint32_t pz = base + (uint32_t)(rd * 16 * S + s * width + warp);
                XRegs xr;
                load_xregs(xr, sm.st, s, r, t, 1);
                ring_wait(sm.ring, pz, w);
                SliceRegs rg;
                const unsigned char* slot = sm.ring.slot(pz);
                load_slice_smem(rg, reinterpret_cast<const uint4*>(slot), reinterpret_cast<const uint4*>(slot + 2048), lane);
                ring_release(sm.ring, pz, lane);
                float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, vv[4];
                compute_slice_x(rg, xr, accS, accB);
                finish_acc4(accS, accB, t, vv);
                tot0 += vv[0]; tot2 += vv[2];
            }
            if (t == 0) {
                const int row_a = (t0 + tl) * 16 + r, row_b = row_a + 8;
                const float la = h2f(f2h(tot0)), lb = h2f(f2h(tot2));
                if (la > best[0] || (la == best[0] && row_a < besti[0])) { best[0] = la; besti[0] = row_a; }
                if (lb > best[0] || (lb == best[0] && row_b < besti[0])) { best[0] = lb; besti[0] = row_b; }
            }
        }
        // the warp's maximum (lanes with t != 0 hold -inf), then the CTA's, then CTA 0 gathers all
        float bv = best[0]; int bi = besti[0];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sm.misc->red16[warp] = bv; sm.misc->redi16[warp] = bi; }
        cbar();
        PS_MARK(a.n_layers, 2);
        if (warp == 0) {
            bv = (lane < PS_CW) ? sm.misc->red16[lane] : -INFINITY; bi = (lane < PS_CW) ? sm.misc->redi16[lane] : 0x7fffffff;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) ll_store(Xw + a.x_off_arg + c, __float_as_uint(bv), (uint32_t)bi, seq);      // read by CTA 0 alone: copy 0 only
            if (c == 0) {
                bv = -INFINITY; bi = 0x7fffffff;
                for (int p = lane; p < g.G; p += 32) {
                    uint32_t d0, d1;
                    ll_load(X + a.x_off_arg + p, seq, d0, d1, w);
                    const float ov = __uint_as_float(d0); const int oi = (int)d1;
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
                if (lane == 0) {
                    // end of the step: the token, the caches' bookkeeping, the next step's sequence number
                    const bool bad = sm.misc->abort != 0;
                    a.out_tok[0] = bad ? 0 : bi;
                    a.tok_in[0] = bad ? 0 : bi;
                    if (a.hist) { const int hp = *a.hist_pos; a.hist[hp % a.hist_cap] = bad ? 0 : bi; *a.hist_pos = (hp + 1) % a.hist_cap; }
                    a.tab.kv_len[slot_id] = kv_len0 + 1;
                    a.tab.parity[slot_id] = side ^ 1;
                    *a.step_seq = seq + 1u;
                    if (tl_cta) tl_cta[a.n_layers * 24 + 3] = ps_now() - t_start;
                }
            }
        }
    }
}

// ---- host side ----
size_t ps_smem_bytes() { return (size_t)PS_SMEM_BYTES; }
int ps_threads() { return PS_THREADS; }

// Whether the one-kernel step can run this geometry on this device, and with how many CTAs: all CTAs must be
// resident together (cooperative launch, one per multiprocessor), and every per-CTA buffer must hold its phase.
bool ps_plan(PsGeom& g, int n_sm) {
    static int configured_dev = -1;
    int dev = 0; cudaGetDevice(&dev);
    if (configured_dev != dev) {
        if (cudaFuncSetAttribute(k_step_persistent, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_BYTES) != cudaSuccess) { cudaGetLastError(); return false; }
        configured_dev = dev;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_step_persistent, PS_THREADS, PS_SMEM_BYTES) != cudaSuccess || per_sm < 1) { cudaGetLastError(); return false; }
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return false;
    g.G = n_sm;
    g.S_h = g.H >> 8; g.S_i = g.I >> 8;
    if (g.H > 2048 || g.valDim > 4096 || g.attn_out > 4096 || g.E > 256 || g.topk > 15) return false;
    const int nsl = g.topk + 1;
    g.gu_spp = g.G / nsl; if (g.gu_spp > g.I / 8) g.gu_spp = g.I / 8;
    if (g.gu_spp < 1) return false;
    const int total_rows = g.Hv * GDN_DV;
    g.rows_per_sm = 4 * ((total_rows + 4 * g.G - 1) / (4 * g.G));
    if (g.rows_per_sm > 32) return false;                          // v_s[32]; also keeps a CTA inside two value heads
    g.router_spr = (g.H * 2 + 2047) / 2048;
    if (g.NH > g.G || g.KV * 64 > g.G * 64) return false;
    // per-CTA maxima: units whose partials are held at once, staged rows of the down phase
    auto ceil_div = [](int x, int y) { return (x + y - 1) / y; };
    const int in_units = ceil_div((g.gdn_in > g.attn_in ? g.gdn_in : g.attn_in) / 16, g.G) * g.S_h;
    const int out_units = ceil_div(g.H / 16, g.G) * ((g.valDim > g.attn_out ? g.valDim : g.attn_out) >> 8);
    const int gu_units = ceil_div(g.I / 8, g.gu_spp) * g.S_h;
    const int down_units = ceil_div(g.H / 16, g.G) * nsl * g.S_i;
    int mx = in_units; if (out_units > mx) mx = out_units; if (gu_units > mx) mx = gu_units; if (down_units > mx) mx = down_units;
    if (mx > PS_RED_UNITS) return false;
    if ((size_t)nsl * ((g.I + 8) * 2 + (g.I >> 6) * 8 * 4) > (size_t)PS_XS_BYTES) return false;
    if (g.E & 7) return false;
    return true;
}

int launch_step_persistent(const PStepArgs& a, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.geom.G); cfg.blockDim = dim3(PS_THREADS); cfg.dynamicSmemBytes = PS_SMEM_BYTES; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    PStepArgs copy = a;
    return (int)cudaLaunchKernelEx(&cfg, k_step_persistent, copy);
}

}  // namespace sl
