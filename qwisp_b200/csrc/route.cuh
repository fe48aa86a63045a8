// route.cuh -- top-k routing of one row by one warp, shared by every kernel that routes.
#pragma once
#include "common.cuh"

namespace sl {

// One warp routes one row.  Restates swift/Sources/QwispCore/SeedlessFusedVerify.swift:180-214
// including the ORDER of its 256-slot halving trees: lane l looks at slots l, l+32, .., l+224, so
// the tree levels 128/64/32 are lane-local and the levels 16..1 are xor-shuffles whose results
// are meaningful in lanes < s -- the same pairs (i, i+s) the reference combines.  Softmax in f32,
// gates rounded to fp16, top-k by k rounds of arg-max on the raw logits (strict > keeps the
// lower slot), fp16 sequential sum of the chosen gates, fp16 divide.
// buf: 2*256 floats + 32 ints of shared memory owned by this warp.  Loops are kept rolled: this
// code runs in one warp of one CTA, so a small instruction footprint matters more than ILP.
// Order of the reference's selection tree (256 slots halved to 128, 64, ... 1, the lower slot of
// each compared pair winning ties): larger logit first, then smaller bit-reversed slot number (the
// last level compares slots 0 and 1, so bit 0 of the slot decides first).  A 24-bit key
// (order-preserving fp16 bits, then 255 - bitreverse8(slot)) has the same order, so k hardware
// warp-max reductions select the same experts in the same sequence.
// SMEM: lrow points to shared memory (plain loads); otherwise to global memory written by other CTAs of a
// running kernel or by an earlier kernel (L1-bypassing loads).
template <bool SMEM>
// early_flag (shared memory, may be null): set to early_value as soon as inds_out is complete, before the gates.
__device__ __noinline__ void route_row_impl(const __half* lrow, int E, int topk, int* inds_out, __half* scores_out, float* buf, int lane,
                                            volatile int* early_flag = nullptr, int early_value = 0) {
    float* lg = buf;
    {   // one 16-byte load per lane covers the 256 slots; shared memory turns it into the slot = j*32+lane order
        uint4 raw = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);      // -inf pairs
        const bool vec = ((E & 7) == 0) && lane * 8 + 8 <= E;     // rows of E halves stay 16-byte aligned only then
        if (vec) raw = SMEM ? reinterpret_cast<const uint4*>(lrow)[lane] : __ldcg(reinterpret_cast<const uint4*>(lrow) + lane);
        const __half* rh = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) lg[lane * 8 + i] = (lane * 8 + i < E) ? h2f(rh[i]) : -INFINITY;
        if (!vec && lane * 8 < E)
            for (int i = 0; i < 8 && lane * 8 + i < E; ++i) lg[lane * 8 + i] = h2f(SMEM ? lrow[lane * 8 + i] : __ldcg(lrow + lane * 8 + i));
    }
    __syncwarp();
    float v0[8];
    unsigned key[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v0[j] = lg[j * 32 + lane]; mx = fmaxf(mx, v0[j]);
        unsigned hb = __half_as_ushort(f2h(v0[j]));                       // exact: the value came from fp16
        if (hb == 0x8000u) hb = 0u;                                       // -0 compares equal to +0
        hb = (hb & 0x8000u) ? (~hb & 0xffffu) : (hb | 0x8000u);
        key[j] = (j * 32 + lane < E) ? ((hb << 8) | (255u - (__brev((unsigned)(j * 32 + lane)) >> 24))) : 0u;
    }
    // Selection first: it needs only the keys, and the chosen experts are what the weight fetch is waiting for.
    int my_id = 0;                                                         // lane k ends up holding the k-th choice
#pragma unroll 1
    for (int k = 0; k < topk; ++k) {
        unsigned best = key[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) best = max(best, key[j]);
        best = __reduce_max_sync(0xffffffffu, best);
        const int slot = (int)(__brev(255u - (best & 0xffu)) >> 24), ol = slot & 31, oj = slot >> 5;
#pragma unroll
        for (int j = 0; j < 8; ++j) if (j == oj && lane == ol) key[j] = 0u;
        if (lane == k) my_id = slot;
    }
    if (lane < topk) inds_out[lane] = my_id;
    if (early_flag) {                                                      // publish the choices before the gate arithmetic
        __syncwarp();
        if (lane == 0) { __threadfence_block(); *early_flag = early_value; }
    }
    mx = warp_max(mx);
    float ex[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { int slot = j * 32 + lane; ex[j] = (slot < E) ? expf(v0[j] - mx) : 0.0f; }
    float r0 = __fadd_rn(ex[0], ex[4]), r1 = __fadd_rn(ex[1], ex[5]), r2 = __fadd_rn(ex[2], ex[6]), r3 = __fadd_rn(ex[3], ex[7]);
    r0 = __fadd_rn(r0, r2); r1 = __fadd_rn(r1, r3);
    r0 = __fadd_rn(r0, r1);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) r0 = __fadd_rn(r0, __shfl_xor_sync(0xffffffffu, r0, s));
    const float Z = __shfl_sync(0xffffffffu, r0, 0);
    float my_ex = 0.f;                                                     // exp of the lane's own choice, fetched from the lane that holds it
#pragma unroll 1
    for (int k = 0; k < topk; ++k) {
        const int id = __shfl_sync(0xffffffffu, my_id, k), ol = id & 31, oj = id >> 5;
        float e_sel = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) if (j == oj) e_sel = ex[j];
        e_sel = __shfl_sync(0xffffffffu, e_sel, ol);
        if (lane == k) my_ex = e_sel;
    }
    // gate of the k-th choice = fp16(exp / Z); the sum runs in fp16 in ascending k, then each is divided by it
    const __half g = f2h(__fdiv_rn(my_ex, Z));
    __half ss = f2h(0.0f);
    for (int k = 0; k < topk; ++k) ss = hadd_rn(ss, __ushort_as_half((unsigned short)__shfl_sync(0xffffffffu, (unsigned)__half_as_ushort(g), k)));
    if (lane < topk) scores_out[lane] = hdiv_rn(g, ss);
    __syncwarp();
}

__device__ __forceinline__ void route_row_warp(const __half* lrow, int E, int topk, int* inds_out, __half* scores_out, float* buf, int lane) {
    route_row_impl<false>(lrow, E, topk, inds_out, scores_out, buf, lane);
}
__device__ __forceinline__ void route_row_smem(const __half* lrow, int E, int topk, int* inds_out, __half* scores_out, float* buf, int lane,
                                               volatile int* early_flag = nullptr, int early_value = 0) {
    route_row_impl<true>(lrow, E, topk, inds_out, scores_out, buf, lane, early_flag, early_value);
}

}  // namespace sl
