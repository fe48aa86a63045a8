// kernels.cu -- the Seedless decode kernels for sm_100a and their launchers.
#include "kernels.h"
#include "mixer_math.cuh"
#include "route.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <array>
#include <map>
#include <string>
#include <vector>

namespace sl {

// multiprocessors of the current device (queried once per device; the launch shapes below are sized by it)
int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static std::atomic<int64_t> g_launches{0};
int64_t kernel_launch_count() { return g_launches.load(); }
#define COUNT_LAUNCH() g_launches.fetch_add(1, std::memory_order_relaxed)

// ---- optional per-kernel timing with CUDA events on the launching stream (eager launches only) ----
struct ProfEntry { const char* tag; cudaEvent_t a, b; double bytes; };
static bool g_prof_on = false;
static std::vector<ProfEntry> g_prof;
struct ProfScope {
    cudaStream_t st; bool on;
    ProfScope(const char* tag, double bytes, cudaStream_t s) : st(s), on(g_prof_on) {
        if (!on) return;
        ProfEntry e{tag, nullptr, nullptr, bytes};
        cudaEventCreate(&e.a); cudaEventCreate(&e.b);
        cudaEventRecord(e.a, st);
        g_prof.push_back(e);
    }
    ~ProfScope() { if (on) cudaEventRecord(g_prof.back().b, st); }
};
void profile_start() { g_prof_on = true; }
void count_launch() { COUNT_LAUNCH(); }
void count_launches(int64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void profile_launch(const char* tag, cudaStream_t st, const std::function<int()>& fn) {
    ProfScope ps(tag, 0.0, st);
    fn();
    COUNT_LAUNCH();
}
// one line per kernel: "tag launches total_ms total_bytes"; stops profiling
int profile_report(char* buf, size_t cap) {
    g_prof_on = false;
    cudaDeviceSynchronize();
    std::map<std::string, std::array<double, 3>> acc;
    for (auto& e : g_prof) {
        float ms = 0.f; cudaEventElapsedTime(&ms, e.a, e.b);
        auto& r = acc[e.tag]; r[0] += 1; r[1] += ms; r[2] += e.bytes;
        cudaEventDestroy(e.a); cudaEventDestroy(e.b);
    }
    g_prof.clear();
    std::string out;
    char line[256];
    for (auto& kv : acc) { snprintf(line, sizeof line, "%s %.0f %.6f %.0f\n", kv.first.c_str(), kv.second[0], kv.second[1], kv.second[2]); out += line; }
    if (out.size() + 1 > cap) return -1;
    memcpy(buf, out.c_str(), out.size() + 1);
    return (int)out.size();
}

// ============================================================================================
// Dense q4 GEMV, split flavour: a CTA holds TPC tiles of 16 weight rows, WPT warps share a tile's
// K/256 slices (see gemv_plan), up to 8 activation rows per pass.  grid (ceil(tiles/TPC), ceil(M/8)).
// Weights are requested before the grid dependency is awaited, so under programmatic dependent
// launch their latency overlaps the tail of the previous kernel.
// ============================================================================================
static void set_pdl(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, bool pdl) {
    if (!pdl) return;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
}
// NW warps per CTA, UPW units per warp; the CTA's NW*UPW units arrive in rounds of 16.
template <int PRO, int EPI, int NW, int UPW>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 2 : 1) k_gemv(DenseArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    const int slices = a.K >> 8, lg = a.lg_slices;
    constexpr int UNITS = NW * UPW, ROUNDS = UNITS / 16;
    const int TPC = UNITS >> lg;
    const int row0 = blockIdx.y * ROWS_PER_PASS;
    const int mr = min(ROWS_PER_PASS, a.M - row0);
    WStage ws; XStage st; float* red; float* fin; int* misc;
    GemvSmem::carve(GemvSmem::carve_w(smem, UNITS, ws), min(a.M, ROWS_PER_PASS), a.K, UNITS, TPC, st, red, fin, misc);
    const int ntiles = (EPI == EPI_SWIGLU) ? a.N / 8 : a.N / 16;
    const int nvu = min(TPC, ntiles - (int)blockIdx.x * TPC) << lg;      // valid units of this CTA
    // The weights do not depend on the kernel before this one: one thread starts their bulk copies
    // into shared memory before the programmatic-launch wait, so they stream in while that kernel
    // finishes and while this CTA stages its activations; they occupy neither registers nor the
    // load/store queue.  Dependents are released only after the wait, so whatever a dependent
    // reads ahead of its own wait was written by a kernel that is complete.
    if (threadIdx.x == (NW - 1) * 32) wstage_issue(ws, a.q.wr, a.q.sr, (size_t)blockIdx.x * TPC << lg, nvu, ROUNDS);   // last warp: least staging work
    StageSrc src{a.x, a.ldx, nullptr, a.nw, a.z, a.ldz, a.eps, a.nw32};
    StageRegs sregs;
    stage_issue_const<PRO>(sregs, src, mr, a.K);
    pdl_wait();
    pdl_launch_dependents();
    stage_issue<PRO>(sregs, src, row0, mr, a.K);
    // the residual value this thread will add in the epilogue (first epilogue iteration) is final already:
    // request it now instead of at the end of the kernel
    __half resid0 = f2h(0.0f);
    if (EPI == EPI_RESID) {
        const int i = threadIdx.x, tl2 = i >> 7, col = (i >> 4) & 7, row = i & 15, tile2 = blockIdx.x * TPC + tl2;
        if (i < TPC * 128 && tile2 < ntiles && col < mr) resid0 = a.y[(size_t)(row0 + col) * a.ldy + tile2 * 16 + row];
    }
    if (blockIdx.y == 0) prefetch_ranges(a.pf, blockIdx.x, gridDim.x);
    stage_finish<PRO>(sregs, st, src, row0, mr, a.K);
    __syncthreads();
    XRegs xr;                                     // the warp's slice is the same for all its units (NW % slices == 0)
    load_xregs(xr, st, warp & (slices - 1), r, t, mr);
#pragma unroll 1
    for (int i = 0; i < UPW; ++i) {
        const int u = warp + NW * i;
        if (u < nvu) {
            if (!mbar_wait_bounded(ws.bar + (u >> 4), 0) && a.err && lane == 0) atomicOr(a.err, 1u);
            SliceRegs rg;
            load_slice_smem(rg, ws.w + (size_t)u * 128, ws.s + (size_t)u * 16, lane);
            float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
            compute_slice_x(rg, xr, accS, accB);
            finish_acc4(accS, accB, t, v);
            store_partial(red, u, lane, v);
        }
    }
    __syncthreads();
    // each output's thread adds the slices' partials itself (ascending order) and writes the result
    if (EPI == EPI_STORE || EPI == EPI_RESID) {
        for (int i = threadIdx.x; i < TPC * 128; i += blockDim.x) {
            int tl2 = i >> 7, col = (i >> 4) & 7, row = i & 15, tile2 = blockIdx.x * TPC + tl2;
            if (tile2 < ntiles && col < mr) {
                size_t idx = (size_t)(row0 + col) * a.ldy + tile2 * 16 + row;
                __half val = f2h(tile_sum(red, tl2, slices, row, col));
                if (EPI == EPI_RESID) val = hadd_rn(i == (int)threadIdx.x ? resid0 : a.y[idx], val);
                a.y[idx] = val;
            }
        }
    } else {   // EPI_SWIGLU
        for (int j = threadIdx.x; j < TPC * 64; j += blockDim.x) {
            int tl2 = j >> 6, col = (j >> 3) & 7, i = j & 7, tile2 = blockIdx.x * TPC + tl2;
            if (tile2 < ntiles && col < mr) {
                __half g = f2h(tile_sum(red, tl2, slices, i, col)), u = f2h(tile_sum(red, tl2, slices, i + 8, col));
                a.y[(size_t)(row0 + col) * a.ldy + tile2 * 8 + i] = swiglu_h(g, u);
            }
        }
    }
}
template <int PRO, int EPI, int NW, int UPW>
static void launch_gemv_t(const DenseArgs& a, const GemvPlan& pl, cudaStream_t st, bool pdl) {
    size_t smem = GemvSmem::wstage_bytes(NW * UPW) + GemvSmem::bytes(a.M < ROWS_PER_PASS ? a.M : ROWS_PER_PASS, a.K, NW * UPW, pl.tpc);
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_gemv<PRO, EPI, NW, UPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); configured = true; }
    int ntiles = EPI == EPI_SWIGLU ? a.N / 8 : a.N / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((ntiles + pl.tpc - 1) / pl.tpc), (unsigned)((a.M + ROWS_PER_PASS - 1) / ROWS_PER_PASS));
    cfg.blockDim = dim3(NW * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    DenseArgs copy = a; copy.lg_slices = pl.lg_slices;
    // profiling tag by role: the in-projection form stores its rows, the out-projection form adds the residual
    ProfScope ps(EPI == EPI_RESID ? "k_gemv_outproj" : "k_gemv_inproj", (double)a.N * a.K * 0.5625 + (double)a.M * (a.K + a.N) * 2, st);
    cudaLaunchKernelEx(&cfg, k_gemv<PRO, EPI, NW, UPW>, copy);
    COUNT_LAUNCH();
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }
template <int PRO>
__global__ void __launch_bounds__(256) k_head(DenseArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    const int slices = a.K >> 8, ntiles = a.N / 16;
    const int row0 = blockIdx.y * ROWS_PER_PASS;
    const int mr = min(ROWS_PER_PASS, a.M - row0);
    XStage st; float* red; float* fin; int* misc;
    GemvSmem::carve(smem, min(a.M, ROWS_PER_PASS), a.K, 1, 1, st, red, fin, misc);      // red: [8 warps][2 rows] values, fin: indices
    const int stride = gridDim.x * nw;
    int tile = blockIdx.x * nw + warp;
    bool have = tile < ntiles;
    SliceRegs cur, nxt;
    const size_t wstep = q4r_w_uint4(a.K), sstep = q4r_s_uint4(a.K);
    auto load = [&](SliceRegs& rg, int tl, int sl_i) { load_slice(rg, a.q.wr + (size_t)tl * wstep, a.q.sr + (size_t)tl * sstep, sl_i, lane); };
    if (have) load(cur, tile, 0);                 // weights: ahead of the programmatic-launch wait
    pdl_wait();
    pdl_launch_dependents();
    if (PRO == PRO_PLAIN) stage_plain(st, a.x, a.ldx, row0, mr, a.K);
    else stage_rmsnorm(st, a.x, a.ldx, a.nw, a.eps, row0, mr, a.K);
    __syncthreads();
    // lane (r, t) sees weight rows r and r+8 of each tile for pass-rows (MMA columns) 2t and 2t+1
    float best[2] = {-INFINITY, -INFINITY}; int besti[2] = {0x7fffffff, 0x7fffffff};
    while (have) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        for (int sidx = 0; sidx < slices; ++sidx) {
            int ns = sidx + 1, ntile = tile;
            if (ns == slices) { ns = 0; ntile = tile + stride; }
            if (ntile < ntiles) load(nxt, ntile, ns);
            float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f};
            compute_slice(cur, st, sidx, r, t, mr, accS, accB);
            float v[4];
            finish_acc4(accS, accB, t, v);
#pragma unroll
            for (int j = 0; j < 4; ++j) tot[j] += v[j];
            cur = nxt;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int col = 2 * t + j;
            if (col < mr) {
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    int row = tile * 16 + r + 8 * hb;
                    __half hv = f2h(tot[2 * hb + j]);
                    if (a.logits) a.logits[(size_t)(row0 + col) * a.N + row] = hv;
                    float lv = h2f(hv);
                    if (better(lv, row, best[j], besti[j])) { best[j] = lv; besti[j] = row; }
                }
            }
        }
        tile += stride; have = tile < ntiles;
    }
    // merge over r (xor 4, 8, 16): lanes 0..3 then hold the warp's maxima of pass-rows 2t, 2t+1
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best[j], off); int oi = __shfl_xor_sync(0xffffffffu, besti[j], off);
            if (better(ov, oi, best[j], besti[j])) { best[j] = ov; besti[j] = oi; }
        }
    int* fini = reinterpret_cast<int*>(fin);
    if (lane < 4) {
        red[warp * 8 + 2 * lane] = best[0]; red[warp * 8 + 2 * lane + 1] = best[1];
        fini[warp * 8 + 2 * lane] = besti[0]; fini[warp * 8 + 2 * lane + 1] = besti[1];
    }
    __syncthreads();
    const int parts = gridDim.x;
    if ((int)threadIdx.x < mr) {
        int col = threadIdx.x; float bv = -INFINITY; int bi = 0x7fffffff;
        for (int w = 0; w < nw; ++w) if (better(red[w * 8 + col], fini[w * 8 + col], bv, bi)) { bv = red[w * 8 + col]; bi = fini[w * 8 + col]; }
        a.pval[(size_t)(row0 + col) * parts + blockIdx.x] = bv;
        a.pidx[(size_t)(row0 + col) * parts + blockIdx.x] = bi;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned total = gridDim.x * gridDim.y;
        unsigned ticket = atomicAdd(a.counter, 1u);
        misc[0] = (ticket == total - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!misc[0]) return;
    __threadfence();
    for (int m = warp; m < a.M; m += nw) {          // one warp per row over the per-CTA partials
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int p = lane; p < parts; p += 32) {
            float lv = __ldcg(a.pval + (size_t)m * parts + p); int li = __ldcg(a.pidx + (size_t)m * parts + p);
            if (better(lv, li, bv, bi)) { bv = lv; bi = li; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, off); int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) a.out_tok[m] = bi;
    }
    if (threadIdx.x == 0) *a.counter = 0u;
}

template <int PRO>
static void launch_head_t(const DenseArgs& a, cudaStream_t st, bool pdl) {
    size_t smem = GemvSmem::bytes(a.M < ROWS_PER_PASS ? a.M : ROWS_PER_PASS, a.K, 1, 1);
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_head<PRO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); configured = true; }
    int ntiles = a.N / 16;
    // one wave of persistent CTAs: as many as are resident at once with this kernel's registers and shared memory
    static int per_sm = 0;
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_head<PRO>, 256, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
        if (per_sm > 3) per_sm = 3;
    }
    int gx = (ntiles + 7) / 8; if (gx > sm_count() * per_sm) gx = sm_count() * per_sm;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)((a.M + ROWS_PER_PASS - 1) / ROWS_PER_PASS));
    cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    DenseArgs copy = a;
    ProfScope ps("k_head", (double)a.N * a.K * 0.5625 + (double)a.M * a.K * 2, st);
    cudaLaunchKernelEx(&cfg, k_head<PRO>, copy);
    COUNT_LAUNCH();
}

// ---- lm_head + greedy argmax with its scratch in a fixed module-scope array (no allocation) ----
// Layout of the array: [0,256) the completion counter, then per-CTA maxima as float
// [HEAD_STATIC_MAX_ROWS][HEAD_STATIC_MAX_PARTS], then their indices as int with the same shape.
#define HEAD_STATIC_MAX_ROWS 8
#define HEAD_STATIC_MAX_PARTS (148 * 3)
#define HEAD_STATIC_BYTES (256 + 2 * HEAD_STATIC_MAX_ROWS * HEAD_STATIC_MAX_PARTS * 4)
static __device__ __align__(256) unsigned char g_head_static_scratch[HEAD_STATIC_BYTES];

int head_static_max_rows() { return HEAD_STATIC_MAX_ROWS; }

// Returns 0, or the cudaError_t of the failing call.  The array's address is looked up once per
// device; nothing here allocates.  The counter is cleared on the stream before every launch, the
// maxima need no clearing because each launch overwrites every entry it later reads.
int launch_head_static(const DenseArgs& in, cudaStream_t st) {
    static unsigned char* base[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!base[dev]) {
        unsigned char* ptr = nullptr;
        err = cudaGetSymbolAddress((void**)&ptr, g_head_static_scratch);
        if (err != cudaSuccess) return (int)err;
        err = cudaFuncSetAttribute(k_head<PRO_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (err != cudaSuccess) return (int)err;
        base[dev] = ptr;
    }
    DenseArgs a = in;
    a.counter = reinterpret_cast<unsigned*>(base[dev]);
    a.pval = reinterpret_cast<float*>(base[dev] + 256);
    a.pidx = reinterpret_cast<int*>(base[dev] + 256 + HEAD_STATIC_MAX_ROWS * HEAD_STATIC_MAX_PARTS * 4);
    const int ntiles = a.N / 16;
    int gx = (ntiles + 7) / 8; if (gx > HEAD_STATIC_MAX_PARTS) gx = HEAD_STATIC_MAX_PARTS;
    err = cudaMemsetAsync(a.counter, 0, sizeof(unsigned), st);
    if (err != cudaSuccess) return (int)err;
    const size_t smem = GemvSmem::bytes(a.M < ROWS_PER_PASS ? a.M : ROWS_PER_PASS, a.K, 1, 1);
    k_head<PRO_PLAIN><<<dim3((unsigned)gx, (unsigned)((a.M + ROWS_PER_PASS - 1) / ROWS_PER_PASS)), 256, smem, st>>>(a);
    return (int)cudaGetLastError();
}

// Gated RMSNorm of the GDN out-projection as a row kernel (prefill mode): one warp per 256 inputs (two heads of
// 128) of one row, the arithmetic of the GEMV prologue (normgate8); out is dense [M][K].
template <int PRO>
__global__ void __launch_bounds__(256) k_normgate_rows(const __half* y, int ldy, const __half* z, int ldz, const __half* nw, const float* nw32,
                                                       float eps, int M, int K, __half* out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, chunks = K >> 8;
    const long u = (long)blockIdx.x * 8 + warp;
    if (u >= (long)M * chunks) return;
    const int row = (int)(u / chunks), k0 = ((int)(u % chunks) << 8) + lane * 8;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(y + (size_t)row * ldy + k0));
    const uint4 zv = __ldcg(reinterpret_cast<const uint4*>(z + (size_t)row * ldz + k0));
    const uint4 wv = *reinterpret_cast<const uint4*>(nw + (k0 & 127));
    *reinterpret_cast<uint4*>(out + (size_t)row * K + k0) = normgate8<PRO>(v, zv, wv, nw32, k0, eps);
}
static void launch_normgate_rows(int pro, const DenseArgs& a, cudaStream_t st) {
    ProfScope ps("k_normgate_rows", (double)a.M * a.K * 6, st);
    const unsigned grid = (unsigned)(((long)a.M * (a.K >> 8) + 7) / 8);
    if (pro == PRO_NORMGATE32) k_normgate_rows<PRO_NORMGATE32><<<grid, 256, 0, st>>>(a.x, a.ldx, a.z, a.ldz, a.nw, a.nw32, a.eps, a.M, a.K, a.norm_scratch);
    else k_normgate_rows<PRO_NORMGATE><<<grid, 256, 0, st>>>(a.x, a.ldx, a.z, a.ldz, a.nw, a.nw32, a.eps, a.M, a.K, a.norm_scratch);
    COUNT_LAUNCH();
}

void launch_dense(int pro, int epi, const DenseArgs& a, cudaStream_t st, bool pdl) {
    if (epi == EPI_ARGMAX) {
        if (pro == PRO_RMSNORM) { launch_head_t<PRO_RMSNORM>(a, st, pdl); return; }
        if (pro == PRO_PLAIN) { launch_head_t<PRO_PLAIN>(a, st, pdl); return; }
    }
    // Prefill mode (a.tc, chosen by the caller per CALL, never by the number of rows): the tcgen05
    // tensor-core GEMM, with the RMSNorm done by a row kernel first.  Every row's result there is
    // independent of how many rows share the call, so a prompt split into chunks in any way gives the
    // same bits; the gated norm of the GDN out-projection runs as a row kernel too.  Every call outside
    // prefill mode uses the GEMV family, which walks the rows in passes of 8.
    if (a.tc && a.N % 16 == 0 && a.K % 256 == 0 && (epi == EPI_STORE || epi == EPI_RESID) &&
        (pro == PRO_PLAIN || a.norm_scratch)) {
        const __half* x = a.x; int ldx = a.ldx;
        if (pro == PRO_RMSNORM) {
            if (a.ldx != a.K) goto gemv_path;                  // the row kernel reads dense rows
            launch_final_norm(a.x, a.nw, a.eps, a.M, a.K, a.norm_scratch, st);
            x = a.norm_scratch; ldx = a.K;
        } else if (pro_is_normgate(pro)) {
            launch_normgate_rows(pro, a, st);
            x = a.norm_scratch; ldx = a.K;
        }
        {
            ProfScope ps("k_gemm_umma", (double)a.N * a.K * 0.5625 + (double)a.M * (a.K + a.N) * 2, st);
            launch_gemm_tc(a.q, a.N, a.K, a.M, x, ldx, a.y, a.ldy, epi == EPI_RESID, a.err, st);
            COUNT_LAUNCH();
        }
        return;
    }
gemv_path:
    if (a.M > ROWS_PER_PASS && launch_dense_rows(pro, epi, a, st)) return;
    const GemvPlan pl = gemv_plan(a.K, epi == EPI_SWIGLU ? a.N / 8 : a.N / 16, 1, sm_count());
#define SL_CASE(P, E)                                                                                       \
    if (pro == P && epi == E) {                                                                             \
        if (pl.upw == 1) launch_gemv_t<P, E, 16, 1>(a, pl, st, pdl);                                        \
        else if (pl.upw == 2) launch_gemv_t<P, E, 16, 2>(a, pl, st, pdl);                                   \
        else launch_gemv_t<P, E, 16, 3>(a, pl, st, pdl);                                                    \
        return;                                                                                             \
    }
    SL_CASE(PRO_PLAIN, EPI_STORE)
    SL_CASE(PRO_PLAIN, EPI_RESID)
    SL_CASE(PRO_RMSNORM, EPI_STORE)
    SL_CASE(PRO_NORMGATE, EPI_RESID)
    SL_CASE(PRO_NORMGATE, EPI_STORE)
    SL_CASE(PRO_NORMGATE32, EPI_RESID)
    SL_CASE(PRO_NORMGATE32, EPI_STORE)
#undef SL_CASE
    fprintf(stderr, "seedless_b200: no dense kernel for prologue %d / epilogue %d\n", pro, epi);
    abort();
}

// ============================================================================================
// Embedding gather and final norm (rows only)
// ============================================================================================
__global__ void k_embed(const __half* embed, const int* tokens, int M, int H, int vocab, __half* h) {
    int m = blockIdx.x;
    int tok = tokens[m];
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint4* src = reinterpret_cast<const uint4*>(embed + (size_t)tok * H);
    uint4* dst = reinterpret_cast<uint4*>(h + (size_t)m * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}
// 4-bit embedding table -> fp16 table, once at load.  Each element is scale * nibble + bias in
// half arithmetic with one rounding, which is what the reference computes per looked-up row
// (embed_rows_q4, SeedlessFusedVerify.swift:556-570); doing it for all rows up front turns
// the per-token lookup into a plain row copy.  One thread per 8 elements (one packed word).
__global__ void k_embed_dequant_q4(const uint32_t* __restrict__ w, const __half* __restrict__ sc, const __half* __restrict__ bi,
                                   __half* __restrict__ out, size_t words, int H) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    size_t row = i / (size_t)(H / 8);
    int kw = (int)(i % (size_t)(H / 8));
    size_t g = row * (size_t)(H / 64) + (size_t)(kw / 8);
    const __half s = sc[g], b = bi[g];
    const uint32_t pack = w[i];
    alignas(16) __half v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __hfma(s, __int2half_rn((int)((pack >> (4 * j)) & 0xFu)), b);
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(v);
}
void launch_embed_dequant_q4(const uint32_t* w, const __half* s, const __half* b, __half* out, int64_t vocab, int H, cudaStream_t st) {
    const size_t words = (size_t)vocab * (size_t)(H / 8);
    const unsigned blocks = (unsigned)((words + 255) / 256);
    k_embed_dequant_q4<<<blocks, 256, 0, st>>>(w, s, b, out, words, H);
}
void launch_embed(const __half* embed, const int* tokens, int M, int H, int vocab, __half* h, cudaStream_t st) {
    ProfScope ps("k_embed", (double)M * H * 4, st);
    k_embed<<<M, 256, 0, st>>>(embed, tokens, M, H, vocab, h);
    COUNT_LAUNCH();
}

// block-wide rmsnorm of one row of width H (multiple of 256, <= 4096) with 256 threads
// xq_row / sx_row (optional): the normed row also in the prepared form of the many-row kernels (paired order + group sums)
__device__ __forceinline__ void block_rmsnorm_row(const __half* src, const __half* w, float eps, int H, __half* dst, float* sm8,
                                                  bool pre = false, uint4 pv = make_uint4(0, 0, 0, 0), uint4 pw = make_uint4(0, 0, 0, 0),
                                                  __half* xq_row = nullptr, float* sx_row = nullptr) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the thread's first 8-element chunk and its weights stay in registers across the reduction,
    // so the common case (H <= 8 * blockDim) touches global memory once
    const int k0 = threadIdx.x * 8;
    uint4 v0 = make_uint4(0, 0, 0, 0), w0 = make_uint4(0, 0, 0, 0);
    if (pre) { v0 = pv; w0 = pw; }
    else if (k0 < H) { v0 = *reinterpret_cast<const uint4*>(src + k0); if (w) w0 = *reinterpret_cast<const uint4*>(w + k0); }
    float ss = 0.f;
    for (int k = k0; k < H; k += blockDim.x * 8) {
        uint4 v = (k == k0) ? v0 : *reinterpret_cast<const uint4*>(src + k);
        const __half2* hh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(hh[i]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) sm8[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += sm8[i];
    float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)H), eps));
    for (int k = k0; k < H; k += blockDim.x * 8) {
        uint4 v = (k == k0) ? v0 : *reinterpret_cast<const uint4*>(src + k);
        const __half* hv = reinterpret_cast<const __half*>(&v);
        uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
        if (w) {
            uint4 wv = (k == k0) ? w0 : *reinterpret_cast<const uint4*>(w + k);
            const __half* wh = reinterpret_cast<const __half*>(&wv);
#pragma unroll
            for (int i = 0; i < 8; ++i) oh[i] = hmul_rn(wh[i], f2h(__fmul_rn(h2f(hv[i]), inv)));
        } else {
            o = v;
        }
        *reinterpret_cast<uint4*>(dst + k) = o;
        if (xq_row) rows_store(xq_row, sx_row, k, o, lane);     // (every thread of the warp is here: H is a multiple of 256)
    }
}
__global__ void k_final_norm(const __half* h, const __half* w, float eps, int H, __half* out, __half* xq, float* sxq) {
    __shared__ float sm8[8];
    block_rmsnorm_row(h + (size_t)blockIdx.x * H, w, eps, H, out + (size_t)blockIdx.x * H, sm8, false, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0),
                      xq ? xq + (size_t)blockIdx.x * H : nullptr, sxq ? sxq + (size_t)blockIdx.x * (H >> 6) : nullptr);
}
// expert-parallel form: every thread also stores the pieces of the normed row it has just written into every rank's gather
// buffer over peer memory, so the rows travel while the router logits are computed; the routing kernel sends the indices
// and raises the flags (its system-scope fence follows these stores in stream order)
__global__ void k_final_norm_ep(const __half* h, const __half* w, float eps, int H, __half* out, EpDispatch epd, int M) {
    __shared__ float sm8[8];
    const int m = blockIdx.x;
    block_rmsnorm_row(h + (size_t)m * H, w, eps, H, out + (size_t)m * H, sm8);
    for (int k = threadIdx.x * 8; k < H; k += blockDim.x * 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(out + (size_t)m * H + k);     // written by this thread
        for (int d = 0; d < epd.sig.world; ++d)
            *reinterpret_cast<uint4*>(epd.pbuf[d] + ((size_t)epd.sig.rank * M + m) * H + k) = v;
    }
}
void launch_final_norm(const __half* h, const __half* w, float eps, int M, int H, __half* out, cudaStream_t st, __half* xq, float* sxq) {
    ProfScope ps("k_final_norm", (double)M * H * 4, st);
    k_final_norm<<<M, 256, 0, st>>>(h, w, eps, H, out, xq, sxq);
    COUNT_LAUNCH();
}
void launch_final_norm_ep(const __half* h, const __half* w, float eps, int M, int H, __half* out, const EpDispatch& epd, cudaStream_t st) {
    ProfScope ps("k_final_norm", (double)M * H * 4, st);
    k_final_norm_ep<<<M, 256, 0, st>>>(h, w, eps, H, out, epd, M);
    COUNT_LAUNCH();
}

// ============================================================================================
// MoE router logits.  fp16 router [E][H]; the dot product follows a fixed order (lane l owns 8
// consecutive inputs of every 256-wide block, sequential f32 accumulate, xor-butterfly over the
// lanes) so that the fp16 logits, and with them the selected experts, are bit-identical to the
// CPU restatement.  The reference's router is the same lane layout over an 8-bit weight
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:384-434).
// grid: E/8 + 1 CTAs of 256 threads (one warp per expert); the last CTA writes the normed rows
// and the shared-expert gate logit.
// ============================================================================================
// MULTI: several rows per call (one warp per row in the norm); the one-row instantiation leaves that code
// out, so it does not compete for registers with the router rows held across the wait
// Q8: the router rows and the shared gate are 8-bit group-64 (the checkpoint's layout).  Lane l owns 8
// consecutive inputs of every 256-wide block, as in the reference's 8-bit GEMV
// (SeedlessMetalForward.swift:378-434): per block accum = sum of x_i * byte_i (i ascending), the lane adds
// scale * accum + (sum of x_i) * bias, lanes are summed by the butterfly.
template <bool MULTI, bool Q8>
__global__ void __launch_bounds__(256, MULTI ? 2 : 1) k_moe_router(RouterArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __half* ps = reinterpret_cast<__half*>(smem);            // [8][H]
    float* sm8 = reinterpret_cast<float*>(ps + 8 * a.H);
    __shared__ int s_last; __shared__ int s_cnt[256]; __shared__ int s_cur[256]; __shared__ int s_off[256];
    __shared__ float s_route[8][512 + 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int nblk = a.H >> 8;                                // <= 16
    const bool tail = (blockIdx.x == gridDim.x - 1);
    const int e = blockIdx.x * 8 + warp;
    // router rows and norm weights do not depend on the kernel before: loaded ahead of the wait
    uint4 pv = make_uint4(0, 0, 0, 0), pw = make_uint4(0, 0, 0, 0);
    if (a.norm_w && tid * 8 < a.H) pw = *reinterpret_cast<const uint4*>(a.norm_w + tid * 8);
    uint4 wreg[16];                                          // fp16 form: 8 halves per block
    uint2 qreg[16]; __half2 sbreg[16];                        // 8-bit form: 8 bytes per block, (scale, bias) of the lane's group
    const bool wvalid = tail ? (warp == 0) : (e < a.E);
    if constexpr (Q8) {
        const uint8_t* qrow = tail ? a.sg_q8 : (a.router_q8 + (size_t)e * a.H);
        const __half* srow = tail ? a.sg_qs : (a.router_qs + (size_t)e * (a.H >> 6));
        const __half* brow = tail ? a.sg_qb : (a.router_qb + (size_t)e * (a.H >> 6));
#pragma unroll
        for (int kb = 0; kb < 16; ++kb) {
            const bool ok = wvalid && kb < nblk;
            qreg[kb] = ok ? *reinterpret_cast<const uint2*>(qrow + kb * 256 + lane * 8) : make_uint2(0, 0);
            sbreg[kb] = ok ? __halves2half2(srow[kb * 4 + (lane >> 3)], brow[kb * 4 + (lane >> 3)]) : __halves2half2(f2h(0.f), f2h(0.f));
        }
    } else {
        const __half* wrow = tail ? a.shared_gate : (a.router + (size_t)e * a.H);
#pragma unroll
        for (int kb = 0; kb < 16; ++kb)
            wreg[kb] = (wvalid && kb < nblk) ? *reinterpret_cast<const uint4*>(wrow + kb * 256 + lane * 8) : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    pdl_launch_dependents();
    if (a.norm_w && tid * 8 < a.H) pv = *reinterpret_cast<const uint4*>(a.h + tid * 8);
    prefetch_ranges(a.pf, blockIdx.x, gridDim.x);
    {   // rows m0 .. m0+7 of this CTA (grid.y walks the row groups)
        const int m0 = blockIdx.y * 8;
        int mr = min(8, a.M - m0);
        __syncthreads();
        if (!MULTI || a.M == 1 || !a.norm_w || (a.H & 255)) {
            for (int c = 0; c < mr; ++c) {
                const __half* src = a.h + (size_t)(m0 + c) * a.ldh;
                if (a.norm_w) block_rmsnorm_row(src, a.norm_w, a.eps, a.H, ps + c * a.H, sm8, m0 + c == 0, pv, pw);
                else for (int k = threadIdx.x * 8; k < a.H; k += blockDim.x * 8) *reinterpret_cast<uint4*>(ps + c * a.H + k) = *reinterpret_cast<const uint4*>(src + k);
            }
        } else if (MULTI && warp < mr) {
            // several rows: one warp per row, the eight rows of a pass side by side.  Same sums in the same
            // order as the block-wide form (per thread 8 elements, a butterfly per 256-chunk, chunks added
            // in ascending order), so the normed rows are identical bit for bit.
            const __half* src = a.h + (size_t)(m0 + warp) * a.ldh;
            uint4 xv[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) xv[c] = (c < nblk) ? *reinterpret_cast<const uint4*>(src + c * 256 + lane * 8) : make_uint4(0, 0, 0, 0);
            float tot = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                if (c < nblk) {
                    const __half2* hh = reinterpret_cast<const __half2*>(&xv[c]);
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(hh[i]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
                    tot += warp_sum(ss);
                }
            }
            const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)a.H), a.eps));
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                if (c < nblk) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(a.norm_w + c * 256 + lane * 8);
                    const __half* hv = reinterpret_cast<const __half*>(&xv[c]);
                    const __half* wh = reinterpret_cast<const __half*>(&wv);
                    uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
                    for (int i = 0; i < 8; ++i) oh[i] = hmul_rn(wh[i], f2h(__fmul_rn(h2f(hv[i]), inv)));
                    *reinterpret_cast<uint4*>(ps + warp * a.H + c * 256 + lane * 8) = o;
                }
            }
        }
        __syncthreads();
        if (tail) {
            for (int i = threadIdx.x; i < mr * a.H / 8; i += blockDim.x) {
                int c = i / (a.H / 8), k = (i - c * (a.H / 8)) * 8;
                *reinterpret_cast<uint4*>(a.p + (size_t)(m0 + c) * a.H + k) = *reinterpret_cast<const uint4*>(ps + c * a.H + k);
            }
        }
        if (wvalid) {
            for (int c = 0; c < mr; ++c) {
                const __half* xrow = ps + c * a.H;
                float acc = 0.f;
#pragma unroll
                for (int kb = 0; kb < 16; ++kb) {
                    if (kb < nblk) {
                        uint4 xv = *reinterpret_cast<const uint4*>(xrow + kb * 256 + lane * 8);
                        const __half* xh = reinterpret_cast<const __half*>(&xv);
                        if constexpr (Q8) {
                            float sum = 0.f, accum = 0.f;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float xf = h2f(xh[i]);
                                const unsigned q = ((i < 4 ? qreg[kb].x : qreg[kb].y) >> (8 * (i & 3))) & 0xffu;
                                sum = __fadd_rn(sum, xf);
                                accum = fmaf(xf, (float)q, accum);                              // product exact in f32
                            }
                            const float2 sb = __half22float2(sbreg[kb]);
                            acc = __fadd_rn(acc, __fadd_rn(__fmul_rn(sb.x, accum), __fmul_rn(sum, sb.y)));
                        } else {
                            const __half* wh = reinterpret_cast<const __half*>(&wreg[kb]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc = fmaf(h2f(xh[i]), h2f(wh[i]), acc);   // product exact in f32
                        }
                    }
                }
                float d = warp_sum(acc);
                if (lane == 0) { if (tail) a.sgl[m0 + c] = f2h(d); else a.logits[(size_t)(m0 + c) * a.E + e] = f2h(d); }
            }
        }
    }
    if (a.no_route) return;                                  // the consumer routes from the logits itself
    // ---- the CTA that finishes last for a group of 8 rows routes those rows (one warp per row), so the groups are
    //      routed side by side; the last of THOSE CTAs then groups the (row, k) pairs of all rows by expert ----
    __threadfence();
    __syncthreads();
    if (tid == 0) { unsigned ticket = atomicAdd(a.group_counter + blockIdx.y, 1u); s_last = (ticket == gridDim.x - 1) ? 1 : 0; }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        const int m = blockIdx.y * 8 + warp;
        if (m < a.M) route_row_warp(a.logits + (size_t)m * a.E, a.E, a.topk, a.inds + m * a.topk, a.scores + m * a.topk, s_route[warp], lane);
    }
    if (tid == 0) a.group_counter[blockIdx.y] = 0u;
    __threadfence();
    __syncthreads();
    if (tid == 0) { unsigned ticket = atomicAdd(a.counter, 1u); s_last = (ticket == gridDim.y - 1) ? 1 : 0; }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *a.counter = 0u;
    __syncthreads();
    if (a.epd.sig.world > 0) {
        // expert-parallel: this CTA sends the rank's normed rows (written by the tail CTAs, complete once the last
        // ticket was drawn) and routing indices into every rank's gather buffers over peer memory, then raises this
        // rank's dispatch flag there; the pair lists are built from the gathered indices by a later kernel
        const EpSignal& sg = a.epd.sig;
        const int nv = a.M * a.H / 8, ni = a.M * a.topk;
        for (int d = 0; d < sg.world; ++d) {
            uint4* dst = reinterpret_cast<uint4*>(a.epd.pbuf[d] + (size_t)sg.rank * a.M * a.H);
            const uint4* src = reinterpret_cast<const uint4*>(a.p);
            for (int i = tid; i < nv; i += 256) dst[i] = __ldcg(src + i);
            int* di = a.epd.ibuf[d] + (size_t)sg.rank * ni;
            for (int i = tid; i < ni; i += 256) di[i] = __ldcg(a.inds + i);
        }
        __threadfence_system();
        __syncthreads();
        if (tid < sg.world) st_release_sys(sg.flags[tid] + sg.rank, ep_seq(sg.ctr, sg.layer, 0));
        return;
    }
    if (a.M == 1) {                                          // one row: its k experts are distinct, slot k = k-th choice
        if (tid < a.topk) {
            a.lists.slot_expert[tid] = __ldcg(a.inds + tid); a.lists.slot_off[tid] = tid; a.lists.slot_cnt[tid] = 1; a.lists.pairs[tid] = tid;
        }
        if (tid == 0) *a.lists.n_active = a.topk;
        return;
    }
    s_cnt[tid] = 0; s_cur[tid] = 0; s_off[tid] = 0;
    __syncthreads();
    const int npairs = a.M * a.topk;
    for (int i = tid; i < npairs; i += 256) atomicAdd(&s_cnt[__ldcg(a.inds + i)], 1);
    __syncthreads();
    if (tid == 0) {
        int slot = 0, off = 0;
        for (int ex = 0; ex < a.E; ++ex)
            if (s_cnt[ex] > 0) {
                a.lists.slot_expert[slot] = ex; a.lists.slot_off[slot] = off; a.lists.slot_cnt[slot] = s_cnt[ex];
                s_off[ex] = off; off += s_cnt[ex]; ++slot;
            }
        *a.lists.n_active = slot;
    }
    __syncthreads();
    for (int i = tid; i < npairs; i += 256) {
        int ex = __ldcg(a.inds + i);
        int pos = atomicAdd(&s_cur[ex], 1);
        a.lists.pairs[s_off[ex] + pos] = i;
    }
}
void launch_router(const RouterArgs& a, cudaStream_t st, bool pdl) {
    size_t smem = (size_t)8 * a.H * 2 + 64;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(k_moe_router<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(k_moe_router<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(k_moe_router<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(k_moe_router<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((a.E + 7) / 8 + 1), (unsigned)((a.M + 7) / 8)); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    RouterArgs copy = a;
    ProfScope ps("k_moe_router", (double)(a.E + 1) * a.H * 2 + (double)a.M * a.H * 4, st);
    const bool q8 = a.router_q8 != nullptr;
    if (a.M == 1) { if (q8) cudaLaunchKernelEx(&cfg, k_moe_router<false, true>, copy); else cudaLaunchKernelEx(&cfg, k_moe_router<false, false>, copy); }
    else { if (q8) cudaLaunchKernelEx(&cfg, k_moe_router<true, true>, copy); else cudaLaunchKernelEx(&cfg, k_moe_router<true, false>, copy); }
    COUNT_LAUNCH();
}

// ============================================================================================
// Routed + shared experts, grouped by expert: every touched expert's weights are read once per
// call and applied to all rows routed to it (8 rows per MMA pass).  Same CTA organisation as the
// split GEMV (TPC tiles per CTA, WPT warps per tile).
// gate/up: grid (ceil((I/8)/TPC), nslots + 1); tile = 8 gate rows + 8 up rows, SwiGLU in the epilogue.
// down:    grid (ceil((H/16)/TPC), nslots + 1).  The last grid.y index is the shared expert (all
//          rows).  The CTA that finishes last for a group of output tiles also does the weighted
//          combine + shared expert + residual for those outputs.
// hbuf / dbuf rows: pair id (row*top_k + k) for routed experts, M*top_k + row for the shared one.
// ============================================================================================
// tile pointers of expert e (or the shared expert) in the repacked slabs
template <bool DOWN>
__device__ __forceinline__ void expert_tile(const ExpertArgs& a, bool shared, int e, int tile, int K, const uint4*& wt, const uint4*& stl) {
    const Q4R& q = DOWN ? (shared ? a.sh_down : a.down) : (shared ? a.sh_gu : a.gu);
    const size_t T = (size_t)e * (DOWN ? a.H / 16 : a.I / 8) + tile;
    wt = q.wr + T * q4r_w_uint4(K); stl = q.sr + T * q4r_s_uint4(K);
}
template <bool DOWN, int UPW>
__global__ void __launch_bounds__(512, 1) k_expert(ExpertArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    const int K = DOWN ? a.I : a.H;
    const int slices = K >> 8, lg = a.lg_slices;
    const int TPC = (16 * UPW) >> lg;
    const int ntiles = DOWN ? a.H / 16 : a.I / 8;
    const int npair = a.M * a.topk;
    // A CTA owns one group of output tiles (blockIdx.x) and walks the expert slots blockIdx.y,
    // blockIdx.y + gridDim.y, ...; slot n_active stands for the shared expert.  With two weight
    // stages the next slot's weights stream in while the current slot is computed.
    XStage st; float* red; float* fin; int* misc;
    const size_t stage_bytes = GemvSmem::wstage_bytes(16 * UPW);
    auto stage_at = [&](int s_) { WStage w; GemvSmem::carve_w(smem + (size_t)s_ * stage_bytes, 16 * UPW, w); return w; };
    GemvSmem::carve(smem + (size_t)a.nstages * stage_bytes, min(a.M, ROWS_PER_PASS), K, 16 * UPW, TPC, st, red, fin, misc);
    const int nvu = min(TPC, ntiles - (int)blockIdx.x * TPC) << lg;      // valid units of this CTA
    const bool issuer = (threadIdx.x == 480);               // last warp: it stages no activations at batch 1
    auto issue = [&](int j, int n_active, int stage) {
        const bool sh = (j == n_active);
        const int e = sh ? 0 : a.lists.slot_expert[j];
        const Q4R& q = DOWN ? (sh ? a.sh_down : a.down) : (sh ? a.sh_gu : a.gu);
        wstage_copy(stage_at(stage), q.wr, q.sr, ((size_t)e * ntiles + (size_t)blockIdx.x * TPC) << lg, nvu, UPW);
    };
    if (issuer) { wstage_init(stage_at(0), UPW); if (a.nstages == 2) wstage_init(stage_at(1), UPW); }
    // What may be read ahead of the programmatic-launch wait: data written two or more kernels back
    // (every kernel releases its dependents only after its own wait).  For the down kernel that
    // covers the router's lists, so its first weights stream into shared memory while gate/up still
    // computes; gate/up follows the router directly, so only the shared expert's weights qualify,
    // and which CTA row takes the shared expert is known ahead of the lists only at batch 1.
    const bool early_shared = !DOWN && a.M == 1 && (int)gridDim.y == a.topk + 1 && blockIdx.y == gridDim.y - 1;
    if (early_shared && issuer) issue((int)gridDim.y - 1, (int)gridDim.y - 1, 0);
    if (!DOWN) { pdl_wait(); pdl_launch_dependents(); }
    const int n_active = *a.lists.n_active;
    const int total = n_active + 1;
    if (!early_shared && (int)blockIdx.y < total && issuer) issue(blockIdx.y, n_active, 0);
    if (DOWN) { pdl_wait(); pdl_launch_dependents(); }
    int it = 0;
    for (int j = blockIdx.y; j < total; j += gridDim.y, ++it) {
        const int stage = (a.nstages == 2) ? (it & 1) : 0;
        const uint32_t parity = (a.nstages == 2) ? ((it >> 1) & 1) : (it & 1);
        if (issuer) {
            // every warp left the previous iteration through a barrier, so its stage may be refilled
            if (a.nstages == 2) { if (j + (int)gridDim.y < total) issue(j + gridDim.y, n_active, stage ^ 1); }
            else if (it > 0) issue(j, n_active, 0);
        }
        const WStage wsc = stage_at(stage);
        const bool shared = (j == n_active);
        const int cnt = shared ? (a.M_shared >= 0 ? a.M_shared : a.M) : a.lists.slot_cnt[j];
        const int off = shared ? 0 : a.lists.slot_off[j];
        for (int c0 = 0; c0 < cnt; c0 += ROWS_PER_PASS) {
            const int mr = min(ROWS_PER_PASS, cnt - c0);
            if (threadIdx.x < ROWS_PER_PASS) {
                int dst = 0, srow = 0;
                if ((int)threadIdx.x < mr) {
                    if (shared) { dst = npair + c0 + threadIdx.x; srow = a.shared_row0 + c0 + threadIdx.x; }
                    else { int pr = a.lists.pairs[off + c0 + threadIdx.x]; dst = pr; srow = pr / a.topk; }
                }
                misc[threadIdx.x] = DOWN ? dst : srow;     // source row of the activations
                misc[8 + threadIdx.x] = dst;               // destination row
            }
            __syncthreads();
            StageSrc src{DOWN ? a.hbuf : a.p, DOWN ? a.I : a.H, misc, nullptr, nullptr, 0, 0.f};
            StageRegs sregs;
            stage_issue<PRO_PLAIN>(sregs, src, 0, mr, K);
            stage_finish<PRO_PLAIN>(sregs, st, src, 0, mr, K);
            __syncthreads();
            XRegs xr;
            load_xregs(xr, st, warp & (slices - 1), r, t, mr);
#pragma unroll 1
            for (int i = 0; i < UPW; ++i) {
                const int u = warp + 16 * i;
                if (u < nvu) {
                    if (c0 == 0 && !mbar_wait_bounded(wsc.bar + i, parity) && a.err && lane == 0) atomicOr(a.err, 1u);
                    SliceRegs rg;
                    load_slice_smem(rg, wsc.w + (size_t)u * 128, wsc.s + (size_t)u * 16, lane);
                    float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
                    compute_slice_x(rg, xr, accS, accB);
                    finish_acc4(accS, accB, t, v);
                    store_partial(red, u, lane, v);
                }
            }
            __syncthreads();
            reduce_tiles(red, fin, nvu >> lg, slices);
            __syncthreads();
            if (DOWN) {
                for (int i = threadIdx.x; i < TPC * 128; i += blockDim.x) {
                    int tl2 = i >> 7, col = (i >> 4) & 7, row = i & 15, tile2 = blockIdx.x * TPC + tl2;
                    if (tile2 < ntiles && col < mr) {
                        const int dst = misc[8 + col];
                        __half* rowp = a.dbuf + (size_t)dst * a.H;
                        if (a.ep_pairs_per_rank > 0 && dst < npair) {       // routed pair in expert-parallel mode: the owner's buffer
                            const int own = dst / a.ep_pairs_per_rank;
                            rowp = a.peer_dbuf[own] + (size_t)(dst - own * a.ep_pairs_per_rank) * a.H;
                        }
                        rowp[tile2 * 16 + row] = f2h(tile_value(fin + tl2 * 128, row, col));
                    }
                }
            } else {
                for (int j2 = threadIdx.x; j2 < TPC * 64; j2 += blockDim.x) {
                    int tl2 = j2 >> 6, col = (j2 >> 3) & 7, i = j2 & 7, tile2 = blockIdx.x * TPC + tl2;
                    if (tile2 < ntiles && col < mr) {
                        __half g = f2h(tile_value(fin + tl2 * 128, i, col)), u = f2h(tile_value(fin + tl2 * 128, i + 8, col));
                        a.hbuf[(size_t)misc[8 + col] * a.I + tile2 * 8 + i] = swiglu_h(g, u);
                    }
                }
            }
            __syncthreads();
        }
        if (!DOWN || a.tile_counter == nullptr) continue;
        // The CTA that finishes last for this group of output tiles combines them for every row:
        // fp16 weighted sum in ascending k (SeedlessFusedVerify.swift:462-471), + sigmoid(gate logit)
        // * shared (:474-484), + residual (SeedlessMetalForward.swift:1024-1028).
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned ticket = atomicAdd(a.tile_counter + blockIdx.x, 1u);
            misc[16] = (ticket == (unsigned)n_active) ? 1 : 0;           // n_active routed slots + the shared expert
        }
        __syncthreads();
        if (!misc[16]) continue;
        __threadfence();
        if (threadIdx.x == 0) a.tile_counter[blockIdx.x] = 0u;
        const int ncols = min(TPC * 16, a.H - blockIdx.x * TPC * 16);
        for (int i = threadIdx.x; i < a.M * ncols; i += blockDim.x) {
            int m = i / ncols, n = blockIdx.x * TPC * 16 + (i - m * ncols);
            __half acc = f2h(0.0f);
            for (int k = 0; k < a.topk; ++k)
                acc = hadd_rn(acc, hmul_rn(__ldcg(a.dbuf + (size_t)(m * a.topk + k) * a.H + n), a.scores[m * a.topk + k]));
            __half res = hadd_rn(acc, hmul_rn(sigmoid_h(a.sgl[m]), __ldcg(a.dbuf + (size_t)(npair + m) * a.H + n)));
            if (a.resid) a.resid[(size_t)m * a.H + n] = hadd_rn(a.resid[(size_t)m * a.H + n], res);
            else a.out[(size_t)m * a.H + n] = res;
        }
    }
    if (DOWN && a.ep_sig.world > 0) {
        // expert-parallel: every CTA makes its peer stores visible system-wide and draws a ticket; the last one
        // raises this rank's combine flag at every peer
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned ticket = atomicAdd(a.ep_sig.ticket, 1u);
            misc[17] = (ticket == gridDim.x * gridDim.y - 1) ? 1 : 0;
            if (misc[17]) *a.ep_sig.ticket = 0u;
        }
        __syncthreads();
        if (misc[17] && (int)threadIdx.x < a.ep_sig.world)
            st_release_sys(a.ep_sig.flags[threadIdx.x] + 8 + a.ep_sig.rank, ep_seq(a.ep_sig.ctr, a.ep_sig.layer, 1));
    }
}
template <bool DOWN, int UPW>
static void launch_expert_t(const ExpertArgs& a, const GemvPlan& pl, int nslots, cudaStream_t st, bool pdl) {
    int K = DOWN ? a.I : a.H;
    int ntiles = DOWN ? a.H / 16 : a.I / 8;
    const int gx = (ntiles + pl.tpc - 1) / pl.tpc;
    int gy = sm_count() / gx; if (gy < 1) gy = 1;
    if (gy > nslots + 1) gy = nslots + 1;                   // one CTA row per slot at batch 1; fewer rows than slots: CTAs walk them
    const int nstages = (gy < nslots + 1) ? 2 : 1;
    size_t smem = nstages * GemvSmem::wstage_bytes(16 * UPW) + GemvSmem::bytes(a.M < ROWS_PER_PASS ? a.M : ROWS_PER_PASS, K, 16 * UPW, pl.tpc);
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_expert<DOWN, UPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); configured = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)gy);
    cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    ExpertArgs copy = a; copy.lg_slices = pl.lg_slices; copy.nstages = nstages;
    ProfScope ps(DOWN ? "k_expert_down" : "k_expert_gateup", 0.0, st);
    cudaLaunchKernelEx(&cfg, k_expert<DOWN, UPW>, copy);
    COUNT_LAUNCH();
}
// ---- batch-1 decode: gate/up + SwiGLU and down + combine of all slots in one launch ----
// grid (G, top_k + 1): CTA (x, y) computes output-tile group x of slot y in both phases (the two
// phases have the same number of tile groups).  Between the phases the 16 CTAs of a slot meet at a
// counter (all CTAs of the grid are resident: one per SM, and dependents are released only after
// every CTA has started), so the down phase reads the slot's complete SwiGLU row.  Both phases'
// weights are requested at the start, so the down weights arrive while gate/up computes.  The wait
// is bounded: after ~4M polls the CTA records the failure and goes on.
template <int UG, int UD>
__global__ void __launch_bounds__(512, 1) k_expert_fused(ExpertArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    const int lg1 = a.lg_slices, lg2 = a.lg_slices2;
    const int sl1 = a.H >> 8, sl2 = a.I >> 8;
    const int TPC1 = (16 * UG) >> lg1, TPC2 = (16 * UD) >> lg2;
    const int nt1 = a.I / 8, nt2 = a.H / 16;
    const int npair = a.topk;                                  // one row
    WStage ws1, ws2; XStage st; float* red; float* fin; int* misc;
    unsigned char* p = GemvSmem::carve_w(smem, 16 * UG, ws1);
    p = GemvSmem::carve_w(p, 16 * UD, ws2);
    constexpr int UM = UG > UD ? UG : UD;
    GemvSmem::carve(p, 1, a.H > a.I ? a.H : a.I, 16 * UM, TPC1 > TPC2 ? TPC1 : TPC2, st, red, fin, misc);
    const int nvu1 = min(TPC1, nt1 - (int)blockIdx.x * TPC1) << lg1, nvu2 = min(TPC2, nt2 - (int)blockIdx.x * TPC2) << lg2;
    const bool issuer = (threadIdx.x == 480);
    const int y = blockIdx.y;
    auto issue = [&](bool sh, int e) {
        const Q4R& q1 = sh ? a.sh_gu : a.gu; const Q4R& q2 = sh ? a.sh_down : a.down;
        wstage_copy(ws1, q1.wr, q1.sr, ((size_t)e * nt1 + (size_t)blockIdx.x * TPC1) << lg1, nvu1, UG);
        wstage_copy(ws2, q2.wr, q2.sr, ((size_t)e * nt2 + (size_t)blockIdx.x * TPC2) << lg2, nvu2, UD);
    };
    if (issuer) { wstage_init(ws1, UG); wstage_init(ws2, UD); }
    __shared__ float s_rbuf[512 + 32];
    __shared__ int s_inds[16];
    __shared__ __half s_scores[16];
    const bool shared = (y == (int)gridDim.y - 1);             // one row: its top_k experts are distinct, slot k = k-th choice
    if (shared && issuer) issue(true, 0);
    pdl_wait();
    pdl_launch_dependents();
    if (a.route_here) {
        // every CTA routes the row itself from the router's logits (one warp, same deterministic procedure in
        // all CTAs) instead of the router kernel ending in a one-CTA routing tail that all CTAs would wait for.
        // The last warp does it (it stages no activations) and starts this slot's weight copies straight away,
        // while the other warps stage the activation row; the barrier after the staging publishes the scores.
        if (warp == 15) {
            route_row_warp(a.rlogits, a.E, a.topk, s_inds, s_scores, s_rbuf, lane);
            __syncwarp();
            if (!shared && lane == 0) issue(false, s_inds[y]);
            if (blockIdx.x == 0 && y == 0 && lane < a.topk) { a.inds_out[lane] = s_inds[lane]; a.scores_out[lane] = s_scores[lane]; }
        }
    } else {
        if ((int)threadIdx.x < a.topk) { s_inds[threadIdx.x] = a.lists.slot_expert[threadIdx.x]; s_scores[threadIdx.x] = a.scores[threadIdx.x]; }
        if (!shared && issuer) issue(false, a.lists.slot_expert[y]);
    }
    const int dst = shared ? npair : y;                        // row of hbuf / dbuf (pair id k, or top_k for the shared expert)
    // ---- phase 1: gate/up + SwiGLU -> hbuf[dst] ----
    {
        StageSrc src{a.p, a.H, nullptr, nullptr, nullptr, 0, 0.f};
        StageRegs sregs;
        stage_issue<PRO_PLAIN>(sregs, src, a.shared_row0, 1, a.H);
        stage_finish<PRO_PLAIN>(sregs, st, src, a.shared_row0, 1, a.H);
        __syncthreads();                                       // the staged row, and the routing of the last warp
        XRegs xr;
        load_xregs(xr, st, warp & (sl1 - 1), r, t, 1);
#pragma unroll 1
        for (int i = 0; i < UG; ++i) {
            const int u = warp + 16 * i;
            if (u < nvu1) {
                if (!mbar_wait_bounded(ws1.bar + i, 0) && a.err && lane == 0) atomicOr(a.err, 1u);
                SliceRegs rg;
                load_slice_smem(rg, ws1.w + (size_t)u * 128, ws1.s + (size_t)u * 16, lane);
                float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
                compute_slice_x(rg, xr, accS, accB);
                finish_acc4(accS, accB, t, v);
                store_partial(red, u, lane, v);
            }
        }
        __syncthreads();
        for (int j2 = threadIdx.x; j2 < TPC1 * 8; j2 += blockDim.x) {
            int tl2 = j2 >> 3, i = j2 & 7, tile2 = blockIdx.x * TPC1 + tl2;
            if (tile2 < nt1) {
                __half g = f2h(tile_sum(red, tl2, sl1, i, 0)), u = f2h(tile_sum(red, tl2, sl1, i + 8, 0));
                a.hbuf[(size_t)dst * a.I + tile2 * 8 + i] = swiglu_h(g, u);
            }
        }
    }
    // ---- the CTAs of this slot meet: every tile group's part of the SwiGLU row is in hbuf ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* arrive = a.slot_sync + y;
        unsigned* leave = a.slot_sync + gridDim.y + y;
        atomicAdd(arrive, 1u);
        bool ok = false;
        for (int spin = 0; spin < (1 << 22); ++spin) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrive) : "memory");
            if (v >= gridDim.x) { ok = true; break; }
        }
        if (!ok && a.err) atomicOr(a.err, 2u);
        // the last one to leave puts both counters back to zero for the next launch
        if (atomicAdd(leave, 1u) == gridDim.x - 1) { *arrive = 0u; *leave = 0u; }
    }
    __syncthreads();
    // ---- phase 2: down -> dbuf[dst], then the last CTA of the tile group combines ----
    {
        StageSrc src{a.hbuf, a.I, nullptr, nullptr, nullptr, 0, 0.f};
        StageRegs sregs;
        stage_issue<PRO_PLAIN>(sregs, src, dst, 1, a.I);
        stage_finish<PRO_PLAIN>(sregs, st, src, dst, 1, a.I);
        __syncthreads();
        XRegs xr;
        load_xregs(xr, st, warp & (sl2 - 1), r, t, 1);
#pragma unroll 1
        for (int i = 0; i < UD; ++i) {
            const int u = warp + 16 * i;
            if (u < nvu2) {
                if (!mbar_wait_bounded(ws2.bar + i, 0) && a.err && lane == 0) atomicOr(a.err, 1u);
                SliceRegs rg;
                load_slice_smem(rg, ws2.w + (size_t)u * 128, ws2.s + (size_t)u * 16, lane);
                float accS[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
                compute_slice_x(rg, xr, accS, accB);
                finish_acc4(accS, accB, t, v);
                store_partial(red, u, lane, v);
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < TPC2 * 16; i += blockDim.x) {
            int tl2 = i >> 4, row = i & 15, tile2 = blockIdx.x * TPC2 + tl2;
            if (tile2 < nt2) a.dbuf[(size_t)dst * a.H + tile2 * 16 + row] = f2h(tile_sum(red, tl2, sl2, row, 0));
        }
    }
    // what the combine needs besides the other CTAs' results is fetched before the ticket, so the CTA that
    // turns out to be last only waits for the expert outputs (column i of the group per thread; TPC2*16 <= 512)
    const int ncols = min(TPC2 * 16, a.H - (int)blockIdx.x * TPC2 * 16);
    const int ncol = blockIdx.x * TPC2 * 16 + threadIdx.x;
    const bool mine = (int)threadIdx.x < ncols;
    __half hres = f2h(0.0f), sgate = f2h(0.0f);
    __half sck[16];
    if (mine) {
        if (a.resid) hres = a.resid[ncol];
        sgate = sigmoid_h(a.sgl[0]);
#pragma unroll
        for (int k = 0; k < 16; ++k) if (k < a.topk) sck[k] = s_scores[k];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned ticket = atomicAdd(a.tile_counter + blockIdx.x, 1u);
        misc[16] = (ticket == gridDim.y - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!misc[16]) return;
    __threadfence();
    if (threadIdx.x == 0) a.tile_counter[blockIdx.x] = 0u;
    if (mine) {
        __half dk[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) if (k < a.topk) dk[k] = __ldcg(a.dbuf + (size_t)k * a.H + ncol);
        const __half dsh = __ldcg(a.dbuf + (size_t)npair * a.H + ncol);
        __half acc = f2h(0.0f);
#pragma unroll
        for (int k = 0; k < 16; ++k) if (k < a.topk) acc = hadd_rn(acc, hmul_rn(dk[k], sck[k]));
        const __half res = hadd_rn(acc, hmul_rn(sgate, dsh));
        if (a.resid) a.resid[ncol] = hadd_rn(hres, res);
        else a.out[ncol] = res;
    }
}
bool expert_fused_applicable(const ExpertArgs& a) {
    if (a.M != 1 || a.slot_sync == nullptr || a.tile_counter == nullptr || a.topk > 16) return false;
    const GemvPlan p1 = gemv_plan(a.H, a.I / 8, a.topk + 1, sm_count()), p2 = gemv_plan(a.I, a.H / 16, a.topk + 1, sm_count());
    const int g1 = (a.I / 8 + p1.tpc - 1) / p1.tpc, g2 = (a.H / 16 + p2.tpc - 1) / p2.tpc;
    if (g1 != g2 || p1.upw != 2 || p2.upw != 1) return false;            // the 2048 -> 512 -> 2048 expert shape
    if (g1 * (a.topk + 1) > sm_count()) return false;                           // every CTA must be resident at once
    return true;
}
bool launch_expert_fused(const ExpertArgs& a, cudaStream_t st, bool pdl) {
    if (!expert_fused_applicable(a)) return false;
    const GemvPlan p1 = gemv_plan(a.H, a.I / 8, a.topk + 1, sm_count()), p2 = gemv_plan(a.I, a.H / 16, a.topk + 1, sm_count());
    const int g1 = (a.I / 8 + p1.tpc - 1) / p1.tpc;
    size_t smem = GemvSmem::wstage_bytes(32) + GemvSmem::wstage_bytes(16) + GemvSmem::bytes(1, a.H > a.I ? a.H : a.I, 32, p1.tpc > p2.tpc ? p1.tpc : p2.tpc);
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_expert_fused<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); configured = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g1, (unsigned)(a.topk + 1));
    cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    ExpertArgs copy = a; copy.lg_slices = p1.lg_slices; copy.lg_slices2 = p2.lg_slices;
    ProfScope ps("k_expert_fused", (double)(a.topk + 1) * 3.0 * a.I * a.H * 0.5625 + (double)(a.topk + 2) * (a.H + a.I) * 2, st);
    cudaLaunchKernelEx(&cfg, k_expert_fused<2, 1>, copy);
    COUNT_LAUNCH();
    return true;
}

// the plan is sized for the batch-1 case (top_k routed experts + the shared one share a wave); the
// combine in the down kernel works on groups of TPC tiles, so tile_counter needs H/16/TPC entries
template <bool DOWN>
static void launch_expert_d(const ExpertArgs& a, int nslots, cudaStream_t st, bool pdl) {
    const GemvPlan pl = gemv_plan(DOWN ? a.I : a.H, DOWN ? a.H / 16 : a.I / 8, a.topk + 1, sm_count());
    if (pl.upw == 1) launch_expert_t<DOWN, 1>(a, pl, nslots, st, pdl);
    else if (pl.upw == 2) launch_expert_t<DOWN, 2>(a, pl, nslots, st, pdl);
    else launch_expert_t<DOWN, 3>(a, pl, nslots, st, pdl);
}
void launch_expert_gateup(const ExpertArgs& a, int nslots, cudaStream_t st, bool pdl) { launch_expert_d<false>(a, nslots, st, pdl); }
void launch_expert_down(const ExpertArgs& a, int nslots, cudaStream_t st, bool pdl) { launch_expert_d<true>(a, nslots, st, pdl); }

// ============================================================================================
// Gated-delta-net core: causal conv1d + SiLU, q/k l2-style norm + scale, beta / decay, the
// recurrent state update and readout, for all rows of a segment in sequence.
// (conv: SeedlessFusedVerify.swift:634-663; prep: :839-938; recurrence: GatedDelta.swift:63-124)
// grid (8 dv-tiles of 16, Hv, nsegs), 128 threads.  The fp32 state tile [16 dv][128 dk] of this
// CTA lives in registers for the whole call: read once from the current ping-pong side, written
// once to the other side.  Conv history likewise goes from one side to the other.
// ============================================================================================
__global__ void __launch_bounds__(128) k_gdn_core(GdnArgs a) {
    __shared__ float q_s[128], k_s[128], v_s[16];
    __shared__ float red_s[8]; __shared__ float gb_s[2];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dvt = blockIdx.x, hv = blockIdx.y;
    const SegDesc seg = a.segs[blockIdx.z];
    const int hk = hv / (a.Hv / a.Hk);
    const int keyDim = a.Hk * GDN_DK, convDim = 2 * keyDim + a.Hv * GDN_DV;
    const int side = a.tab.parity[seg.slot];
    const float* S_in = a.tab.gdn_state + (size_t)seg.slot * a.tab.state_stride_stream + (size_t)side * a.tab.state_stride_side +
                        (size_t)a.gdn_index * a.tab.state_stride_layer + ((size_t)hv * GDN_DV + dvt * 16) * GDN_DK;
    float* S_out = a.tab.gdn_state + (size_t)seg.slot * a.tab.state_stride_stream + (size_t)(side ^ 1) * a.tab.state_stride_side +
                   (size_t)a.gdn_index * a.tab.state_stride_layer + ((size_t)hv * GDN_DV + dvt * 16) * GDN_DK;
    const __half* hist_in = a.tab.conv_hist + (size_t)seg.slot * a.tab.hist_stride_stream + (size_t)side * a.tab.hist_stride_side +
                            (size_t)a.gdn_index * a.tab.hist_stride_layer;
    __half* hist_out = a.tab.conv_hist + (size_t)seg.slot * a.tab.hist_stride_stream + (size_t)(side ^ 1) * a.tab.hist_stride_side +
                       (size_t)a.gdn_index * a.tab.hist_stride_layer;
    // state rows of this warp: 4 rows, lane owns dk 4*lane .. 4*lane+3
    // the state was written a whole step ago: loaded ahead of the programmatic-launch wait
    float4 S[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) S[i] = *reinterpret_cast<const float4*>(S_in + (size_t)(warp * 4 + i) * GDN_DK + lane * 4);
    // also ahead of the wait: conv weights, decay parameters (cold in HBM once per token) and the three
    // history rows of this thread's channels (written a step ago)
    const int ch_q = hk * GDN_DK + tid, ch_k = keyDim + hk * GDN_DK + tid;
    const int ch_v = 2 * keyDim + hv * GDN_DV + dvt * 16 + (tid & 15);
    const float4 wq = *reinterpret_cast<const float4*>(a.conv_w + (size_t)ch_q * 4);
    const float4 wk = *reinterpret_cast<const float4*>(a.conv_w + (size_t)ch_k * 4);
    const float4 wv = *reinterpret_cast<const float4*>(a.conv_w + (size_t)ch_v * 4);
    const float A_log_h = a.A_log[hv], dt_bias_h = a.dt_bias[hv];
    float hq[CONV_K - 1], hkk[CONV_K - 1], hvv[CONV_K - 1];
#pragma unroll
    for (int j = 0; j < CONV_K - 1; ++j) {
        hq[j] = h2f(hist_in[(size_t)j * convDim + ch_q]);
        hkk[j] = h2f(hist_in[(size_t)j * convDim + ch_k]);
        hvv[j] = h2f(hist_in[(size_t)j * convDim + ch_v]);
    }
    pdl_wait();
    pdl_launch_dependents();

    auto xval = [&](int idx, int ch) -> float {               // row idx of [hist(3) | rows of the segment]
        if (idx < CONV_K - 1) {
            const float* hsel = (ch == ch_q) ? hq : ((ch == ch_k) ? hkk : hvv);
            return (idx == 0) ? hsel[0] : ((idx == 1) ? hsel[1] : hsel[2]);
        }
        return h2f(a.inproj[(size_t)(seg.row0 + idx - (CONV_K - 1)) * a.ld + ch]);
    };
    auto conv = [&](int tt, int ch, float4 w) -> float {
        return gdn_conv_silu(xval(tt + 0, ch), xval(tt + 1, ch), xval(tt + 2, ch), xval(tt + 3, ch), w);
    };
    for (int tt = 0; tt < seg.nrows; ++tt) {
        const int row = seg.row0 + tt;
        float qc = conv(tt, ch_q, wq), kc = conv(tt, ch_k, wk);
        if (tid < 16) v_s[tid] = conv(tt, ch_v, wv);
        float sq = warp_sum(qc * qc), sk = warp_sum(kc * kc);
        if (lane == 0) { red_s[warp] = sq; red_s[4 + warp] = sk; }
        if (tid == 0) {
            __half bh = a.inproj[(size_t)row * a.ld + convDim + a.Hv * GDN_DV + hv];
            __half ah = a.inproj[(size_t)row * a.ld + convDim + a.Hv * GDN_DV + a.Hv + hv];
            gdn_gate(bh, ah, A_log_h, dt_bias_h, gb_s[0], gb_s[1]);
        }
        __syncthreads();
        float iq = gdn_head_inv(red_s[0], red_s[1], red_s[2], red_s[3], a.eps);
        float ik = gdn_head_inv(red_s[4], red_s[5], red_s[6], red_s[7], a.eps);
        q_s[tid] = gdn_scale_q(qc, iq);
        k_s[tid] = gdn_scale_k(kc, ik);
        __syncthreads();
        const float g = gb_s[0], beta = gb_s[1];
        const float4 kq = *reinterpret_cast<const float4*>(k_s + lane * 4);
        const float4 qq = *reinterpret_cast<const float4*>(q_s + lane * 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 s = S[i];
            const float o = gdn_row_step(s, g, kq, qq, v_s[warp * 4 + i], beta);
            S[i] = s;
            if (lane == 0) a.y[(size_t)row * (a.Hv * GDN_DV) + hv * GDN_DV + dvt * 16 + warp * 4 + i] = f2h(o);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(S_out + (size_t)(warp * 4 + i) * GDN_DK + lane * 4) = S[i];
    // new conv history = last three rows of [hist | rows]; q/k channels by one CTA per key head
    const bool owner_qk = (dvt == 0) && (hv % (a.Hv / a.Hk) == 0);
    for (int j = 0; j < CONV_K - 1; ++j) {
        int idx = seg.nrows + j;
        if (owner_qk) {
            hist_out[(size_t)j * convDim + ch_q] = f2h(xval(idx, ch_q));
            hist_out[(size_t)j * convDim + ch_k] = f2h(xval(idx, ch_k));
        }
        if (tid < 16) hist_out[(size_t)j * convDim + ch_v] = f2h(xval(idx, ch_v));
    }
}
// ---- segments of many rows (prompt chunks, verify rows): the same arithmetic in two kernels ----
// k_gdn_prep   everything that does not depend on the state, for all rows side by side: conv + SiLU of every channel, the
//              q/k norms and scales, decay and beta, the conv history the call leaves.  grid (Hk + Hv, M), 128 threads:
//              CTAs [0, Hk) own a key head's q and k channels, CTAs [Hk, Hk + Hv) a value head's v channels and gates.
// k_gdn_scan   the recurrence alone, rows of a segment in sequence, the operands of 32 rows at a time staged in shared
//              memory by cp.async one chunk ahead.
//              Same grid and state ownership as k_gdn_core.
// Every value is formed by the same functions in the same order as in k_gdn_core, so the outputs and the state are
// identical bit for bit; the split only removes the per-row latency chain (and the 16-fold recomputation of q / k).
__global__ void __launch_bounds__(128) k_gdn_prep(GdnArgs a) {
    __shared__ float red_s[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m = blockIdx.y;
    const SegDesc seg = a.segs[a.row_seg[m]];
    const int tt = m - seg.row0;
    const int keyDim = a.Hk * GDN_DK, valDim = a.Hv * GDN_DV, convDim = 2 * keyDim + valDim;
    const int side = a.tab.parity[seg.slot];
    const __half* hist_in = a.tab.conv_hist + (size_t)seg.slot * a.tab.hist_stride_stream + (size_t)side * a.tab.hist_stride_side +
                            (size_t)a.gdn_index * a.tab.hist_stride_layer;
    __half* hist_out = a.tab.conv_hist + (size_t)seg.slot * a.tab.hist_stride_stream + (size_t)(side ^ 1) * a.tab.hist_stride_side +
                       (size_t)a.gdn_index * a.tab.hist_stride_layer;
    auto xval = [&](int idx, int ch) -> float {               // row idx of [hist(3) | rows of the segment]
        if (idx < CONV_K - 1) return h2f(hist_in[(size_t)idx * convDim + ch]);
        return h2f(a.inproj[(size_t)(seg.row0 + idx - (CONV_K - 1)) * a.ld + ch]);
    };
    auto conv = [&](int ch) -> float {
        const float4 w = *reinterpret_cast<const float4*>(a.conv_w + (size_t)ch * 4);
        return gdn_conv_silu(xval(tt + 0, ch), xval(tt + 1, ch), xval(tt + 2, ch), xval(tt + 3, ch), w);
    };
    const bool last = (tt == seg.nrows - 1);
    if ((int)blockIdx.x < a.Hk) {
        const int hk = blockIdx.x, ch_q = hk * GDN_DK + tid, ch_k = keyDim + hk * GDN_DK + tid;
        const float qc = conv(ch_q), kc = conv(ch_k);
        const float sq = warp_sum(qc * qc), sk = warp_sum(kc * kc);
        if (lane == 0) { red_s[warp] = sq; red_s[4 + warp] = sk; }
        __syncthreads();
        const float iq = gdn_head_inv(red_s[0], red_s[1], red_s[2], red_s[3], a.eps);
        const float ik = gdn_head_inv(red_s[4], red_s[5], red_s[6], red_s[7], a.eps);
        a.qk[(size_t)m * 2 * keyDim + hk * GDN_DK + tid] = f2h(gdn_scale_q(qc, iq));              // exact: the value is an fp16 product
        a.qk[(size_t)m * 2 * keyDim + keyDim + hk * GDN_DK + tid] = f2h(gdn_scale_k(kc, ik));
        if (last)
            for (int j = 0; j < CONV_K - 1; ++j) {
                hist_out[(size_t)j * convDim + ch_q] = f2h(xval(seg.nrows + j, ch_q));
                hist_out[(size_t)j * convDim + ch_k] = f2h(xval(seg.nrows + j, ch_k));
            }
    } else {
        const int hv = blockIdx.x - a.Hk, ch_v = 2 * keyDim + hv * GDN_DV + tid;
        a.vc[(size_t)m * valDim + hv * GDN_DV + tid] = f2h(conv(ch_v));                            // exact: conv + SiLU is rounded to fp16
        if (tid == 0) {
            const __half bh = a.inproj[(size_t)m * a.ld + convDim + valDim + hv];
            const __half ah = a.inproj[(size_t)m * a.ld + convDim + valDim + a.Hv + hv];
            float g, beta;
            gdn_gate(bh, ah, a.A_log[hv], a.dt_bias[hv], g, beta);
            a.gb[(size_t)m * a.Hv + hv] = make_float2(g, beta);
        }
        if (last)
            for (int j = 0; j < CONV_K - 1; ++j) hist_out[(size_t)j * convDim + ch_v] = f2h(xval(seg.nrows + j, ch_v));
    }
}
constexpr int GS_CH = 32;                                    // rows per staged chunk
__device__ __forceinline__ void gs_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gs_cp8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__global__ void __launch_bounds__(128) k_gdn_scan(GdnArgs a) {
    // operands of 32 rows at a time, two buffers: q | k of the key head, the 16 v values of this CTA's state rows, (decay, beta)
    __shared__ __align__(16) __half qk_s[2][GS_CH][2 * GDN_DK];
    __shared__ __align__(16) __half v_s[2][GS_CH][16];
    __shared__ __align__(8) float2 gb_s[2][GS_CH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dvt = blockIdx.x, hv = blockIdx.y;
    const SegDesc seg = a.segs[blockIdx.z];
    const int hk = hv / (a.Hv / a.Hk);
    const int keyDim = a.Hk * GDN_DK, valDim = a.Hv * GDN_DV;
    const int side = a.tab.parity[seg.slot];
    const float* S_in = a.tab.gdn_state + (size_t)seg.slot * a.tab.state_stride_stream + (size_t)side * a.tab.state_stride_side +
                        (size_t)a.gdn_index * a.tab.state_stride_layer + ((size_t)hv * GDN_DV + dvt * 16) * GDN_DK;
    float* S_out = a.tab.gdn_state + (size_t)seg.slot * a.tab.state_stride_stream + (size_t)(side ^ 1) * a.tab.state_stride_side +
                   (size_t)a.gdn_index * a.tab.state_stride_layer + ((size_t)hv * GDN_DV + dvt * 16) * GDN_DK;
    float4 S[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) S[i] = *reinterpret_cast<const float4*>(S_in + (size_t)(warp * 4 + i) * GDN_DK + lane * 4);
    auto stage = [&](int c, int b) {
        const int t0 = c * GS_CH, n = min(GS_CH, seg.nrows - t0);
        for (int i = tid; i < n * 32; i += 128) {                                    // q, k: 16 + 16 pieces of 16 bytes per row
            const int r = i >> 5, p = i & 31;
            const size_t row = (size_t)(seg.row0 + t0 + r);
            gs_cp16(&qk_s[b][r][p * 8], a.qk + row * 2 * keyDim + (p < 16 ? 0 : keyDim) + hk * GDN_DK + (p & 15) * 8);
        }
        for (int i = tid; i < n * 2; i += 128) {
            const int r = i >> 1, p = i & 1;
            gs_cp16(&v_s[b][r][p * 8], a.vc + (size_t)(seg.row0 + t0 + r) * valDim + hv * GDN_DV + dvt * 16 + p * 8);
        }
        for (int i = tid; i < n; i += 128) gs_cp8(&gb_s[b][i], a.gb + (size_t)(seg.row0 + t0 + i) * a.Hv + hv);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto h4 = [](uint2 u) -> float4 {
        const __half2 lo = *reinterpret_cast<const __half2*>(&u.x), hi = *reinterpret_cast<const __half2*>(&u.y);
        const float2 a2 = __half22float2(lo), b2 = __half22float2(hi);
        return make_float4(a2.x, a2.y, b2.x, b2.y);
    };
    const int nchunks = (seg.nrows + GS_CH - 1) / GS_CH;
    stage(0, 0);
    for (int c = 0; c < nchunks; ++c) {
        const int b = c & 1;
        if (c + 1 < nchunks) { stage(c + 1, b ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int t0 = c * GS_CH, n = min(GS_CH, seg.nrows - t0);
        for (int r = 0; r < n; ++r) {
            const float4 qq = h4(*reinterpret_cast<const uint2*>(&qk_s[b][r][lane * 4]));
            const float4 kq = h4(*reinterpret_cast<const uint2*>(&qk_s[b][r][GDN_DK + lane * 4]));
            const float4 vv = h4(*reinterpret_cast<const uint2*>(&v_s[b][r][warp * 4]));
            const float2 gb = gb_s[b][r];
            const float vs[4] = {vv.x, vv.y, vv.z, vv.w};
            // the warp's four rows together: their two butterfly sums share shuffles (warp_sum4), same additions as gdn_row_step()
            const float kvz = warp_sum4(gdn_decay_dot(S[0], gb.x, kq), gdn_decay_dot(S[1], gb.x, kq), gdn_decay_dot(S[2], gb.x, kq),
                                        gdn_decay_dot(S[3], gb.x, kq), lane);
            float op[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float kv = __shfl_sync(0xffffffffu, kvz, 8 * i);
                const float delta = (vs[i] - kv) * gb.y;
                op[i] = gdn_update_dot(S[i], kq, delta, qq);
            }
            const float oz = warp_sum4(op[0], op[1], op[2], op[3], lane);
            if ((lane & 7) == 0)
                a.y[(size_t)(seg.row0 + t0 + r) * valDim + hv * GDN_DV + dvt * 16 + warp * 4 + (lane >> 3)] = f2h(oz);
        }
        __syncthreads();                       // the buffer is refilled by the next iteration's stage()
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(S_out + (size_t)(warp * 4 + i) * GDN_DK + lane * 4) = S[i];
}
void launch_gdn_rows(const GdnArgs& a, int M, int nsegs, cudaStream_t st) {
    {
        ProfScope ps("k_gdn_prep", (double)M * (2 * a.Hk * GDN_DK + a.Hv * GDN_DV) * 4, st);
        k_gdn_prep<<<dim3((unsigned)(a.Hk + a.Hv), (unsigned)M), 128, 0, st>>>(a);
        COUNT_LAUNCH();
    }
    ProfScope ps("k_gdn_scan", (double)nsegs * a.Hv * GDN_DV * GDN_DK * 8, st);
    k_gdn_scan<<<dim3(8, (unsigned)a.Hv, (unsigned)nsegs), 128, 0, st>>>(a);
    COUNT_LAUNCH();
}
void launch_gdn_core(const GdnArgs& a, int nsegs, cudaStream_t st, bool pdl) {
    dim3 grid(8, a.Hv, nsegs);
    ProfScope ps("k_gdn_core", (double)nsegs * a.Hv * GDN_DV * GDN_DK * 8, st);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(128); cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    GdnArgs copy = a;
    cudaLaunchKernelEx(&cfg, k_gdn_core, copy);
    COUNT_LAUNCH();
}

// ============================================================================================
// Attention: q/k RMSNorm + partial NeoX RoPE + KV append; split-KV GQA decode; combine + gate.
// KV arena: pages [page][attn layer][K|V][kv head][page_size][256] fp16, K stored post-RoPE.
// (prep: SeedlessFusedVerify.swift:1183-1360; attention: SeedlessMetalForward.swift:4922-4989;
//  output gate: SeedlessMetalForward.swift:1012-1022)
// ============================================================================================
// grid (NH + 2*KV, M), 32 threads: one warp per (row, head); lane owns dims 8*lane..8*lane+7
__global__ void __launch_bounds__(32) k_attn_prep(AttnArgs a) {
    const int m = blockIdx.y, hidx = blockIdx.x, lane = threadIdx.x;
    const int slot = a.segs[a.row_seg[m]].slot;
    const int pos = row_position(a, m);
    const __half* rowp = a.inproj + (size_t)m * a.ld;
    if (hidx >= a.NH + a.KV) {                               // V copy
        int kvh = hidx - a.NH - a.KV;
        const __half* src = rowp + a.NH * 2 * ATT_D + a.KV * ATT_D + kvh * ATT_D;
        __half* dst = kv_ptr(a, slot, pos, 1, kvh);
        reinterpret_cast<uint4*>(dst)[lane] = reinterpret_cast<const uint4*>(src)[lane];
        return;
    }
    const bool isq = hidx < a.NH;
    const __half* src = isq ? (rowp + (size_t)hidx * 2 * ATT_D) : (rowp + a.NH * 2 * ATT_D + (hidx - a.NH) * ATT_D);
    const __half* w = isq ? a.q_norm : a.k_norm;
    uint4 v = reinterpret_cast<const uint4*>(src)[lane];
    uint4 wv = reinterpret_cast<const uint4*>(w)[lane];
    const __half* vh = reinterpret_cast<const __half*>(&v);
    const __half* wh = reinterpret_cast<const __half*>(&wv);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { float f = h2f(vh[i]); ss = fmaf(f, f, ss); }
    ss = warp_sum(ss);
    float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), a.eps));
    float nv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) nv[i] = h2f(hmul_rn(wh[i], f2h(__fmul_rn(h2f(vh[i]), inv))));
    // rotate dims [0,64): pairs (d, d+32); lanes 0..3 hold d<32, lanes 4..7 hold d+32
    float other[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, nv[i], 4);
    uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
    const float fpos = (float)pos;
    const float lnb = logf(a.theta);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int d = lane * 8 + i;
        if (d >= ROPE_D) { oh[i] = f2h(nv[i]); continue; }
        int ii = (d < 32) ? d : (d - 32);
        float freq = expf(-2.0f * (float)ii / (float)ROPE_D * lnb);
        float ang = fpos * freq;
        float sn, cs; sincosf(ang, &sn, &cs);
        float x0 = (d < 32) ? nv[i] : other[i], x1 = (d < 32) ? other[i] : nv[i];
        oh[i] = f2h((d < 32) ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs));
    }
    if (isq) reinterpret_cast<uint4*>(a.qrot + ((size_t)m * a.NH + hidx) * ATT_D)[lane] = o;
    else reinterpret_cast<uint4*>(kv_ptr(a, slot, pos, 0, hidx - a.NH))[lane] = o;
}
void launch_attn_prep(const AttnArgs& a, cudaStream_t st) {
    dim3 grid(a.NH + 2 * a.KV, a.M);
    ProfScope ps("k_attn_prep", 0.0, st);
    k_attn_prep<<<grid, 32, 0, st>>>(a);
    COUNT_LAUNCH();
}

// ---- one-kernel attention: (optional) q/k prep + split-KV decode + merge of the splits ----
// norm + partial rotation of one 256-wide head held as 8 values per lane; returns the fp16 values
__device__ __forceinline__ uint4 norm_rope_head(const __half* src, const __half* w, float eps, float theta, int pos, int lane) {
    uint4 v = reinterpret_cast<const uint4*>(src)[lane];
    uint4 wv = reinterpret_cast<const uint4*>(w)[lane];
    const __half* vh = reinterpret_cast<const __half*>(&v);
    const __half* wh = reinterpret_cast<const __half*>(&wv);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { float f = h2f(vh[i]); ss = fmaf(f, f, ss); }
    ss = warp_sum(ss);
    float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 256.0f), eps));
    float nv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) nv[i] = h2f(hmul_rn(wh[i], f2h(__fmul_rn(h2f(vh[i]), inv))));
    float other[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, nv[i], 4);
    uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
    const float fpos = (float)pos;
    const float lnb = logf(theta);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int d = lane * 8 + i;
        if (d >= ROPE_D) { oh[i] = f2h(nv[i]); continue; }
        int ii = (d < 32) ? d : (d - 32);
        float freq = expf(-2.0f * (float)ii / (float)ROPE_D * lnb);
        float ang = fpos * freq;
        float sn, cs; sincosf(ang, &sn, &cs);
        float x0 = (d < 32) ? nv[i] : other[i], x1 = (d < 32) ? other[i] : nv[i];
        oh[i] = f2h((d < 32) ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs));
    }
    return o;
}
// grid (nsplit, KV heads, M), 256 threads, dynamic shared memory 8*8*256 floats.
// prep != 0 (every row is the only row of its stream in this launch): each CTA norms and rotates its
// 8 query heads itself, and the CTA whose key range holds the row's own position also makes that
// position's K and V, stores them in the arena and uses them from shared memory.  prep == 0: q and
// the arena were written by k_attn_prep.  Either way the CTA that finishes last for a (row, kv head)
// merges the splits, normalises, rounds to fp16 and applies the sigmoid output gate.
__global__ void __launch_bounds__(256) k_attn_fused(AttnArgs a, int prep, unsigned* counters) {
    extern __shared__ __align__(16) float sm_acc[];           // [8 warps][8 heads][256]
    __shared__ float sm_m[8][ATT_G], sm_l[8][ATT_G];
    __shared__ __align__(16) __half sq[ATT_G][ATT_D];
    __shared__ __align__(16) __half sk[ATT_D], sv[ATT_D];
    __shared__ int s_last;
    __shared__ float s_cs[32], s_sn[32];
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Ahead of the programmatic-launch wait: everything that does not depend on this step's in-projection.
    // Stream lengths and page tables were written before the step; with prep != 0 every position below the
    // row's own was stored in an earlier step, so the warp's first keys and values can already be in flight.
    const int slot = a.segs[a.row_seg[m]].slot;
    const int pos_m = row_position(a, m);
    const int N = pos_m + 1;
    int chunk, used, p0, p1;
    attn_split_range(N, a.nsplit, split, chunk, used, p0, p1);
    if (split >= used) { pdl_wait(); pdl_launch_dependents(); return; }
    const bool own = prep && (pos_m >= p0) && (pos_m < p1);
    const __half* rowp = a.inproj + (size_t)m * a.ld;
    uint4 kcur = make_uint4(0, 0, 0, 0), vcur = make_uint4(0, 0, 0, 0);
    const int first = p0 + warp;
    const bool early_kv = prep && first < p1 && first != pos_m;
    if (early_kv) {
        kcur = reinterpret_cast<const uint4*>(kv_ptr(a, slot, first, 0, kvh))[lane];
        vcur = reinterpret_cast<const uint4*>(kv_ptr(a, slot, first, 1, kvh))[lane];
    }
    if (prep && threadIdx.x < 32) rope_table_entry(a.theta, pos_m, threadIdx.x, s_cs[threadIdx.x], s_sn[threadIdx.x]);
    pdl_wait();
    pdl_launch_dependents();
    if (prep) {
        __syncthreads();                                      // the rotation table
        uint4 qo = norm_rope_head_tab(reinterpret_cast<const uint4*>(rowp + (size_t)(kvh * ATT_G + warp) * 2 * ATT_D)[lane], a.q_norm, a.eps, s_cs, s_sn, lane);
        reinterpret_cast<uint4*>(sq[warp])[lane] = qo;
        if (own && warp == 1) {
            uint4 ko = norm_rope_head_tab(reinterpret_cast<const uint4*>(rowp + a.NH * 2 * ATT_D + kvh * ATT_D)[lane], a.k_norm, a.eps, s_cs, s_sn, lane);
            reinterpret_cast<uint4*>(sk)[lane] = ko;
            reinterpret_cast<uint4*>(kv_ptr(a, slot, pos_m, 0, kvh))[lane] = ko;
        }
        if (own && warp == 2) {
            uint4 vo = reinterpret_cast<const uint4*>(rowp + a.NH * 2 * ATT_D + a.KV * ATT_D + kvh * ATT_D)[lane];
            reinterpret_cast<uint4*>(sv)[lane] = vo;
            reinterpret_cast<uint4*>(kv_ptr(a, slot, pos_m, 1, kvh))[lane] = vo;
        }
    } else {
        reinterpret_cast<uint4*>(sq[warp])[lane] = reinterpret_cast<const uint4*>(a.qrot + ((size_t)m * a.NH + kvh * ATT_G + warp) * ATT_D)[lane];
    }
    __syncthreads();
    const float scale = 0.0625f;                              // 256^-0.5
    float q[ATT_G][8];
#pragma unroll
    for (int g = 0; g < ATT_G; ++g) {
        uint4 qv = reinterpret_cast<const uint4*>(sq[g])[lane];
        const __half* qh = reinterpret_cast<const __half*>(&qv);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[g][i] = scale * h2f(qh[i]);
    }
    float mx[ATT_G], l[ATT_G], acc[ATT_G][8];
#pragma unroll
    for (int g = 0; g < ATT_G; ++g) { mx[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f; }
    // keys of this warp: first, first + 8, ...; the next key's K and V are requested before the current one is used
    auto load_kv = [&](int pos, uint4& kk, uint4& vv) {
        if (own && pos == pos_m) { kk = reinterpret_cast<const uint4*>(sk)[lane]; vv = reinterpret_cast<const uint4*>(sv)[lane]; }
        else {
            kk = reinterpret_cast<const uint4*>(kv_ptr(a, slot, pos, 0, kvh))[lane];
            vv = reinterpret_cast<const uint4*>(kv_ptr(a, slot, pos, 1, kvh))[lane];
        }
    };
    if (!early_kv && first < p1) load_kv(first, kcur, vcur);
    for (int pos = first; pos < p1; pos += 8) {
        uint4 knext = make_uint4(0, 0, 0, 0), vnext = make_uint4(0, 0, 0, 0);
        if (pos + 8 < p1) load_kv(pos + 8, knext, vnext);
        const __half* kh = reinterpret_cast<const __half*>(&kcur);
        const __half* vh = reinterpret_cast<const __half*>(&vcur);
        float kf[8], vf[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { kf[i] = h2f(kh[i]); vf[i] = h2f(vh[i]); }
#pragma unroll
        for (int g = 0; g < ATT_G; ++g) attn_key_step(q[g], kf, vf, mx[g], l[g], acc[g]);
        kcur = knext; vcur = vnext;
    }
    // ---- merge the 8 warps: all heads at once through shared memory ----
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < ATT_G; ++g) { sm_m[warp][g] = mx[g]; sm_l[warp][g] = l[g]; }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < ATT_G; ++g) {
        float m8[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) m8[w] = sm_m[w][g];
        const float gm = attn_warps_max(m8);
        float f = (mx[g] == -INFINITY) ? 0.f : __expf(mx[g] - gm);
        float4 lo = make_float4(acc[g][0] * f, acc[g][1] * f, acc[g][2] * f, acc[g][3] * f);
        float4 hi = make_float4(acc[g][4] * f, acc[g][5] * f, acc[g][6] * f, acc[g][7] * f);
        float4* dst = reinterpret_cast<float4*>(sm_acc + ((size_t)warp * ATT_G + g) * ATT_D + lane * 8);
        dst[0] = lo; dst[1] = hi;
    }
    __syncthreads();
    {
        const int d = threadIdx.x;                            // 256 threads = 256 dims
        float* po = a.part_o + (((size_t)m * a.NH + kvh * ATT_G) * a.nsplit + split) * ATT_D;
#pragma unroll
        for (int g = 0; g < ATT_G; ++g) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) o += sm_acc[((size_t)w * ATT_G + g) * ATT_D + d];
            po[(size_t)g * a.nsplit * ATT_D + d] = o;
        }
        if (d < ATT_G) {
            const int g = d;
            float m8[8], l8[8];
            for (int w = 0; w < 8; ++w) { m8[w] = sm_m[w][g]; l8[w] = sm_l[w][g]; }
            const float gm = attn_warps_max(m8);
            const float ls = attn_warps_lsum(m8, l8, gm);
            float* pml = a.part_ml + (((size_t)m * a.NH + kvh * ATT_G + g) * a.nsplit + split) * 2;
            pml[0] = gm; pml[1] = ls;
        }
    }
    // ---- the CTA that finishes last for this (row, kv head) merges the splits ----
    // (the output gate of this warp's head does not depend on the other CTAs: fetched before the ticket)
    const uint4 gvv = reinterpret_cast<const uint4*>(rowp + (size_t)(kvh * ATT_G + warp) * 2 * ATT_D + ATT_D)[lane];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned ticket = atomicAdd(counters + m * a.KV + kvh, 1u);
        s_last = (ticket == (unsigned)used - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        const int g = warp, h = kvh * ATT_G + g;
        const float* po = a.part_o + ((size_t)m * a.NH + h) * a.nsplit * ATT_D;
        const float* pml = a.part_ml + ((size_t)m * a.NH + h) * a.nsplit * 2;
        const uint4 outv = attn_merge_splits(used, lane, gvv,
            [&](int sp, float4& x0, float4& x1) { const float4* src = reinterpret_cast<const float4*>(po + (size_t)sp * ATT_D + lane * 8); x0 = __ldcg(src); x1 = __ldcg(src + 1); },
            [&](int sp) { return __ldcg(reinterpret_cast<const float2*>(pml) + sp); });
        reinterpret_cast<uint4*>(a.gated + ((size_t)m * a.NH + h) * ATT_D)[lane] = outv;
    }
    if (threadIdx.x == 0) counters[m * a.KV + kvh] = 0u;
}
void launch_attn_fused(const AttnArgs& a, bool prep, unsigned* counters, cudaStream_t st, bool pdl) {
    static bool configured = false;
    const size_t smem = (size_t)8 * ATT_G * ATT_D * sizeof(float);
    if (!configured) { cudaFuncSetAttribute(k_attn_fused, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); configured = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.nsplit, (unsigned)a.KV, (unsigned)a.M);
    cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    set_pdl(cfg, attr, pdl);
    AttnArgs copy = a; int p = prep ? 1 : 0;
    ProfScope ps("k_attn_fused", 0.0, st);
    cudaLaunchKernelEx(&cfg, k_attn_fused, copy, p, counters);
    COUNT_LAUNCH();
}


// ---- test hook: a bounded wait that runs out ----
// One CTA waits, with the same routine the weight stages use but a limit of a thousand polls, on an
// mbarrier that nothing ever arms, and reports the way the real kernels do: it sets a bit in the error
// word and returns.  Nothing faults and nothing hangs; the host sees the code at its next synchronisation.
__global__ void k_wait_probe(unsigned* err) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait_bounded(&bar, 0, 1000)) atomicOr(err, 4u);
}
void launch_wait_probe(unsigned* err, cudaStream_t st) { k_wait_probe<<<1, 32, 0, st>>>(err); COUNT_LAUNCH(); }

// ============================================================================================
// End of a step: advance cache lengths, flip GDN ping-pong sides, feed greedy tokens back as
// the next step's input and append them to the device-side history (chained steps).
// ============================================================================================
__global__ void k_step_end(StepEndArgs a) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a.nsegs) {
        SegDesc s = a.segs[i];
        a.tab.kv_len[s.slot] += s.nrows;
        a.tab.parity[s.slot] ^= 1;
    }
    if (a.out_tok && i < a.M) {
        int tk = a.out_tok[i];
        if (a.tok_in) a.tok_in[i] = tk;
        if (a.hist) a.hist[(*a.hist_pos + i) % a.hist_cap] = tk;
    }
    __syncthreads();
    if (a.hist && a.out_tok && i == 0) *a.hist_pos = (*a.hist_pos + a.M) % a.hist_cap;
}
void launch_step_end(const StepEndArgs& a, cudaStream_t st) {
    int n = a.nsegs > a.M ? a.nsegs : a.M;
    if (n > 1024) n = 1024;      // one block: history position is updated after every thread has used it
    ProfScope ps("k_step_end", 0.0, st);
    k_step_end<<<1, n < 32 ? 32 : n, 0, st>>>(a);
    COUNT_LAUNCH();
}

}  // namespace sl
