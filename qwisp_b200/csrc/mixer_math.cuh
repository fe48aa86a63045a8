// mixer_math.cuh -- the arithmetic of the two token mixers (gated delta net, full attention), written once
// and shared by every kernel that runs them, so that the per-phase kernels and the one-kernel decode step
// produce the same bits: each function fixes the operation order of one piece of the reference's math.
// (conv: swift/Sources/QwispCore/SeedlessFusedVerify.swift:634-663; prep: :839-938; recurrence:
//  GatedDelta.swift:63-124; attention prep: SeedlessFusedVerify.swift:1183-1360; attention:
//  SeedlessMetalForward.swift:4922-4989; output gate: SeedlessMetalForward.swift:1012-1022)
#pragma once
#include "common.cuh"

namespace sl {

constexpr int ATT_G = 8;     // query heads per kv head handled together (attn_heads / attn_kv_heads must equal it)

// ---- gated delta net ----
// causal depthwise conv over [hist0, hist1, hist2, x] (f32 accumulate in tap order), SiLU, rounded to fp16
__device__ __forceinline__ float gdn_conv_silu(float x0, float x1, float x2, float x3, float4 w) {
    float acc = 0.f;
    acc = __fadd_rn(acc, __fmul_rn(x0, w.x));
    acc = __fadd_rn(acc, __fmul_rn(x1, w.y));
    acc = __fadd_rn(acc, __fmul_rn(x2, w.z));
    acc = __fadd_rn(acc, __fmul_rn(x3, w.w));
    return h2f(f2h(__fmul_rn(acc, sigmoid_f(acc))));
}
// decay g = exp(-exp(A_log) * softplus(a + dt_bias)) in f32, beta = sigmoid(b) in fp16
__device__ __forceinline__ void gdn_gate(__half bh, __half ah, float A_log_h, float dt_bias_h, float& g, float& beta) {
    beta = h2f(sigmoid_h(bh));
    float xa = h2f(ah) + dt_bias_h;
    float sp = fmaxf(xa, 0.0f) + logf(1.0f + expf(-fabsf(xa)));
    g = expf(-expf(A_log_h) * sp);
}
// inverse rms of a 128-wide head from the four 32-lane partial sums of squares (added left to right)
__device__ __forceinline__ float gdn_head_inv(float r0, float r1, float r2, float r3, float eps) {
    return __frsqrt_rn(__fadd_rn(__fdiv_rn(r0 + r1 + r2 + r3, 128.0f), eps));
}
// q <- fp16(1/128) * fp16(q * inv), k <- fp16(128^-0.5) * fp16(k * inv), as f32 values of the fp16 results
__device__ __forceinline__ float gdn_scale_q(float qc, float iq) {
    const float invScale = 0.08838834764831845f;             // 128^-0.5
    return h2f(hmul_rn(f2h(invScale * invScale), f2h(__fmul_rn(qc, iq))));
}
__device__ __forceinline__ float gdn_scale_k(float kc, float ik) {
    const float invScale = 0.08838834764831845f;
    return h2f(hmul_rn(f2h(invScale), f2h(__fmul_rn(kc, ik))));
}
// One state row (one dv) of one token, the row spread over a warp (lane owns dk 4*lane .. 4*lane+3):
// S <- S*g;  kv = S.k;  delta = (v - kv)*beta;  S += k*delta;  returns o = S.q (the same value in every lane)
// The two lane-local halves, shared by the one-row form below and the four-rows-at-once form of k_gdn_scan:
__device__ __forceinline__ float gdn_decay_dot(float4& s, float g, float4 kq) {
    s.x *= g; s.y *= g; s.z *= g; s.w *= g;
    return s.x * kq.x + s.y * kq.y + s.z * kq.z + s.w * kq.w;
}
__device__ __forceinline__ float gdn_update_dot(float4& s, float4 kq, float delta, float4 qq) {
    s.x = fmaf(kq.x, delta, s.x); s.y = fmaf(kq.y, delta, s.y); s.z = fmaf(kq.z, delta, s.z); s.w = fmaf(kq.w, delta, s.w);
    return s.x * qq.x + s.y * qq.y + s.z * qq.z + s.w * qq.w;
}
__device__ __forceinline__ float gdn_row_step(float4& s, float g, float4 kq, float4 qq, float v, float beta) {
    const float kv = warp_sum(gdn_decay_dot(s, g, kq));
    const float delta = (v - kv) * beta;
    return warp_sum(gdn_update_dot(s, kq, delta, qq));
}
// Butterfly sums of FOUR values per lane at once: the additions are those of four warp_sum() calls (partners at lane
// distance 16, 8, 4, 2, 1, in that order; an addition's operands may be swapped, which changes nothing), but the first
// two levels hand each value to a different quarter of the warp, so 6 shuffles do the work of 20.  On return the lanes
// 8i .. 8i+7 hold the total of value i.
__device__ __forceinline__ float warp_sum4(float a, float b, float c, float d, int lane) {
    const bool hi = (lane & 16) != 0;
    const float r0 = __shfl_xor_sync(0xffffffffu, hi ? a : c, 16), r1 = __shfl_xor_sync(0xffffffffu, hi ? b : d, 16);
    const float x = (hi ? c : a) + r0, y = (hi ? d : b) + r1;           // lanes < 16: values a, b; lanes >= 16: c, d
    const bool b3 = (lane & 8) != 0;
    float z = (b3 ? y : x) + __shfl_xor_sync(0xffffffffu, b3 ? x : y, 8);
    z += __shfl_xor_sync(0xffffffffu, z, 4);
    z += __shfl_xor_sync(0xffffffffu, z, 2);
    z += __shfl_xor_sync(0xffffffffu, z, 1);
    return z;
}

// ---- attention ----
// cos / sin of the 32 rotation angles of one position
__device__ __forceinline__ void rope_table_entry(float theta, int pos, int i, float& cs, float& sn) {
    const float lnb = logf(theta);
    const float freq = expf(-2.0f * (float)i / (float)ROPE_D * lnb);
    const float ang = (float)pos * freq;
    sincosf(ang, &sn, &cs);
}
// RMSNorm (weight w) + partial NeoX rotation of one 256-wide head held as 8 values per lane, angles from a
// table (tab_cs / tab_sn [32]); returns the fp16 values
// (v: the lane's 8 values of the head)
__device__ __forceinline__ uint4 norm_rope_head_tab(uint4 v, const __half* w, float eps, const float* tab_cs, const float* tab_sn, int lane) {
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
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int d = lane * 8 + i;
        if (d >= ROPE_D) { oh[i] = f2h(nv[i]); continue; }
        int ii = (d < 32) ? d : (d - 32);
        const float cs = tab_cs[ii], sn = tab_sn[ii];
        float x0 = (d < 32) ? nv[i] : other[i], x1 = (d < 32) ? other[i] : nv[i];
        oh[i] = f2h((d < 32) ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs));
    }
    return o;
}
// the key range of split `split` for a row that attends to N keys: chunks are multiples of 32 keys
__device__ __forceinline__ void attn_split_range(int N, int nsplit, int split, int& chunk, int& used, int& p0, int& p1) {
    chunk = 32 * ((N + 32 * nsplit - 1) / (32 * nsplit));
    used = (N + chunk - 1) / chunk;
    p0 = split * chunk; p1 = min(N, p0 + chunk);
}
// one key for one query head: online softmax in f32 (q already scaled; the lane's 8 of the 256 dims)
__device__ __forceinline__ void attn_key_step(const float q[8], const float kf[8], const float vf[8], float& mx, float& l, float acc[8]) {
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sc = fmaf(q[i], kf[i], sc);
    sc = warp_sum(sc);
    float nm = fmaxf(mx, sc);
    float factor = __expf(mx - nm), es = __expf(sc - nm);
    mx = nm; l = l * factor + es;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(acc[i], factor, es * vf[i]);
}
// merge of the 8 key-warps of a split for one head: the maximum, and the rescaled normaliser
__device__ __forceinline__ float attn_warps_max(const float m8[8]) {
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) gm = fmaxf(gm, m8[w]);
    return gm;
}
__device__ __forceinline__ float attn_warps_lsum(const float m8[8], const float l8[8], float gm) {
    float ls = 0.f;
    for (int w = 0; w < 8; ++w) ls += (m8[w] == -INFINITY) ? 0.f : l8[w] * __expf(m8[w] - gm);
    return ls;
}
// Merge of the splits of one (row, head) by one warp: part_o [used][256] f32, part_ml [used][2] f32 (both read
// with the loader ld_f / ld_f2 the caller provides), output gate values gvv (8 halves of this lane) ->
// 8 gated fp16 outputs of this lane.  used <= 64.
template <typename LoadF4, typename LoadF2>
__device__ __forceinline__ uint4 attn_merge_splits(int used, int lane, uint4 gvv, LoadF4 ld_o, LoadF2 ld_ml) {
    float msv[2], lsv[2], fv[2];                          // two splits per lane
    float gm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int sp = j * 32 + lane;
        msv[j] = -INFINITY; lsv[j] = 0.f;
        if (sp < used) { float2 ml = ld_ml(sp); msv[j] = ml.x; lsv[j] = ml.y; }
        gm = fmaxf(gm, msv[j]);
    }
    gm = warp_max(gm);
    float tot = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) { fv[j] = (msv[j] == -INFINITY) ? 0.f : __expf(msv[j] - gm); tot += lsv[j] * fv[j]; }
    tot = warp_sum(tot);
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int sp = 0; sp < used; ++sp) {
        float f = __shfl_sync(0xffffffffu, (sp < 32) ? fv[0] : fv[1], sp & 31);
        float4 x0, x1;
        ld_o(sp, x0, x1);
        o[0] = fmaf(x0.x, f, o[0]); o[1] = fmaf(x0.y, f, o[1]); o[2] = fmaf(x0.z, f, o[2]); o[3] = fmaf(x0.w, f, o[3]);
        o[4] = fmaf(x1.x, f, o[4]); o[5] = fmaf(x1.y, f, o[5]); o[6] = fmaf(x1.z, f, o[6]); o[7] = fmaf(x1.w, f, o[7]);
    }
    const __half* gh = reinterpret_cast<const __half*>(&gvv);
    uint4 outv; __half* oh = reinterpret_cast<__half*>(&outv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        __half out = f2h(tot == 0.f ? o[i] : o[i] / tot);
        oh[i] = hmul_rn(out, sigmoid_h(gh[i]));
    }
    return outv;
}

}  // namespace sl
