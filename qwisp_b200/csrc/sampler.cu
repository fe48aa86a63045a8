// sampler.cu -- speculative-sampling rows on the device: per verify row a categorical draw by
// Gumbel-max over the (optionally nucleus-truncated) logits, the same draw with the draft token
// excluded, and the accept test coin < p(draft).  Only three int32 per row leave the device.
// Behaviour follows the reference's kernel (swift/Sources/QwispCore/SamplerGPU.swift:39-156):
// counter-based hash noise keyed by (seed, position + row, token), temperature as 1/T (<= 0 means
// greedy with first-index-wins ties, identical to the argmax path), top-p through a 1024-bucket
// histogram of fixed-point softmax weights over the scaled gap (gmax - L)/T.
//
// exp and log are evaluated by the small deterministic routines below (IEEE add / multiply /
// divide only, no fused contraction), so the CPU restatement used by the tests reproduces every
// draw and every accept flag bit for bit; their ~1e-7 relative error is irrelevant for sampling.
#include "kernels.h"

namespace sl {

__device__ __forceinline__ float det_expf(float x) {           // x <= 0
    if (x < -87.0f) return 0.0f;
    const float n = rintf(__fmul_rn(x, 1.44269504f));
    float r = __fsub_rn(x, __fmul_rn(n, 0.693145751953125f));
    r = __fsub_rn(r, __fmul_rn(n, 1.42860682e-6f));
    float p = 1.0f / 720.0f;
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 120.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 24.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 6.0f);
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    return __fmul_rn(p, __int_as_float(((int)n + 127) << 23));
}
__device__ __forceinline__ float det_logf(float a) {           // a > 0, normal
    int bits = __float_as_int(a);
    int e = ((bits >> 23) & 255) - 127;
    float m = __int_as_float((bits & 0x007fffff) | 0x3f800000);
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float f = __fsub_rn(m, 1.0f);
    const float s = __fdiv_rn(f, __fadd_rn(2.0f, f));
    const float z = __fmul_rn(s, s);
    float p = 1.0f / 9.0f;
    p = __fadd_rn(__fmul_rn(p, z), 1.0f / 7.0f);
    p = __fadd_rn(__fmul_rn(p, z), 0.2f);
    p = __fadd_rn(__fmul_rn(p, z), 1.0f / 3.0f);
    p = __fadd_rn(__fmul_rn(p, z), 1.0f);
    const float lm = __fmul_rn(__fmul_rn(2.0f, s), p);
    const float fe = (float)e;
    return __fadd_rn(__fmul_rn(fe, 0.693145751953125f), __fadd_rn(lm, __fmul_rn(fe, 1.42860682e-6f)));
}
__device__ __forceinline__ uint32_t qhash(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t h = a * 0x9E3779B1u + 0x165667B1u;
    h ^= b + 0x9E3779B9u + (h << 6) + (h >> 2);
    h ^= c + 0x9E3779B9u + (h << 6) + (h >> 2);
    h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
    return h;
}
__device__ __forceinline__ float u01(uint32_t h) { return fmaxf(__fmul_rn((float)(h >> 8), 1.0f / 16777216.0f), 1e-7f); }

constexpr int SAMP_T = 1024;          // threads per row
constexpr int SAMP_BINS = 1024;
constexpr float SAMP_SPAN = 40.0f;

// block-wide sum in a fixed order: per-thread partials, xor butterfly inside each warp, warps added in ascending order
__device__ __forceinline__ float block_sum_fixed(float v, float* sm32) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, s));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm32[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < SAMP_T / 32; ++w) tot = __fadd_rn(tot, sm32[w]);
    __syncthreads();
    return tot;
}
__device__ __forceinline__ bool better_si(float s, int i, float bs, int bi) { return s > bs || (s == bs && i < bi); }

// adj: optional [V] f32 penalties / bias added to every row's logits before anything else looks at them
// (the reference's LADJ(v) = float(row[v]) + logitAdj[v], SamplerGPU.swift:41,69); nullptr = none.
__global__ void __launch_bounds__(SAMP_T) k_sample_rows(const __half* logits, const float* adj, const int* draft, int* samp_full, int* samp_resid, int* accept,
                                                        float invT, int V, uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, float top_p) {
    __shared__ float sm32[32];
    __shared__ float s_fs[32], s_rs[32]; __shared__ int s_fi[32], s_ri[32];
    __shared__ unsigned hist[SAMP_BINS];
    __shared__ float s_lthr;
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __half* row = logits + (size_t)m * V;
    const int d = draft ? draft[m] : -1;
    const bool greedy = invT <= 0.0f;
    const uint32_t salt = seed_hi ^ (base_pos + (uint32_t)m);
    auto ladj = [&](int v) -> float { const float L = h2f(row[v]); return adj ? __fadd_rn(L, adj[v]) : L; };
    // pass 1: maximum (adjusted) logit
    float mx = -INFINITY;
    for (int v = tid; v < V; v += SAMP_T) mx = fmaxf(mx, ladj(v));
    mx = warp_max(mx);
    if (lane == 0) sm32[warp] = mx;
    __syncthreads();
    float gmax = -INFINITY;
    for (int w = 0; w < SAMP_T / 32; ++w) gmax = fmaxf(gmax, sm32[w]);
    __syncthreads();
    const bool do_top_p = !greedy && top_p < 0.999f;
    float lthr = -INFINITY, znuc = 0.f;
    if (!greedy) {
        if (do_top_p) { for (int b = tid; b < SAMP_BINS; b += SAMP_T) hist[b] = 0u; __syncthreads(); }
        const float bin_w = SAMP_SPAN / (float)SAMP_BINS;
        float z = 0.f;
        for (int v = tid; v < V; v += SAMP_T) {
            const float g = __fmul_rn(__fsub_rn(gmax, ladj(v)), invT);
            const float w = det_expf(-g);
            z = __fadd_rn(z, w);
            if (do_top_p) {
                const float q = __fdiv_rn(g, bin_w);
                const unsigned b = (q >= (float)(SAMP_BINS - 1)) ? (unsigned)(SAMP_BINS - 1) : (unsigned)q;
                atomicAdd(&hist[b], (unsigned)__fmul_rn(w, 8192.0f));
            }
        }
        znuc = block_sum_fixed(z, sm32);
        if (do_top_p) {
            if (tid == 0) {
                unsigned total = 0; for (int b = 0; b < SAMP_BINS; ++b) total += hist[b];
                const unsigned target = (unsigned)__fmul_rn(top_p, (float)total);
                unsigned cum = 0; int bstar = SAMP_BINS - 1;
                for (int b = 0; b < SAMP_BINS; ++b) { cum += hist[b]; if (cum >= target) { bstar = b; break; } }
                s_lthr = __fsub_rn(gmax, __fdiv_rn(__fmul_rn((float)(bstar + 1), bin_w), invT));
            }
            __syncthreads();
            lthr = s_lthr;
            float zn = 0.f;
            for (int v = tid; v < V; v += SAMP_T) { const float L = ladj(v); if (L >= lthr) zn = __fadd_rn(zn, det_expf(__fmul_rn(__fsub_rn(L, gmax), invT))); }
            znuc = block_sum_fixed(zn, sm32);
        }
    }
    // Gumbel-max over the nucleus: full, and excluding the draft token
    float fs = -INFINITY, rs = -INFINITY; int fi = 0x7fffffff, ri = 0x7fffffff;
    for (int v = tid; v < V; v += SAMP_T) {
        const float L = ladj(v);
        if (do_top_p && L < lthr) continue;
        float score = L;
        if (!greedy) {
            const float u = u01(qhash(seed_lo, salt, (uint32_t)v));
            score = __fsub_rn(__fmul_rn(L, invT), det_logf(-det_logf(u)));
        }
        if (better_si(score, v, fs, fi)) { fs = score; fi = v; }
        if (v != d && better_si(score, v, rs, ri)) { rs = score; ri = v; }
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        float os = __shfl_xor_sync(0xffffffffu, fs, s); int oi = __shfl_xor_sync(0xffffffffu, fi, s);
        if (better_si(os, oi, fs, fi)) { fs = os; fi = oi; }
        os = __shfl_xor_sync(0xffffffffu, rs, s); oi = __shfl_xor_sync(0xffffffffu, ri, s);
        if (better_si(os, oi, rs, ri)) { rs = os; ri = oi; }
    }
    if (lane == 0) { s_fs[warp] = fs; s_fi[warp] = fi; s_rs[warp] = rs; s_ri[warp] = ri; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SAMP_T / 32; ++w) {
            if (better_si(s_fs[w], s_fi[w], fs, fi)) { fs = s_fs[w]; fi = s_fi[w]; }
            if (better_si(s_rs[w], s_ri[w], rs, ri)) { rs = s_rs[w]; ri = s_ri[w]; }
        }
        samp_full[m] = fi;
        samp_resid[m] = (d < 0) ? fi : ri;
        float p_draft = 0.f;
        if (d >= 0) {
            if (greedy) p_draft = (d == fi) ? 1.0f : 0.0f;
            else {
                const float Ld = ladj(d);
                if (!do_top_p || Ld >= lthr) p_draft = __fdiv_rn(det_expf(__fmul_rn(__fsub_rn(Ld, gmax), invT)), znuc);
            }
        }
        const float coin = u01(qhash(seed_lo, salt, 0x9999AAAAu));
        accept[m] = (coin < p_draft) ? 1 : 0;
    }
}
void launch_sample_rows(const __half* logits, const float* adj, const int* draft, int* samp_full, int* samp_resid, int* accept, int M, int V,
                        float invT, float top_p, uint32_t seed_lo, uint32_t seed_hi, uint32_t base_pos, cudaStream_t st) {
    k_sample_rows<<<M, SAMP_T, 0, st>>>(logits, adj, draft, samp_full, samp_resid, accept, invT, V, seed_lo, seed_hi, base_pos, top_p);
}

}  // namespace sl
