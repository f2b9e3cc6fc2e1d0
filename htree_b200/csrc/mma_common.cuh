// Pieces shared by the tensor-core forward and backward kernels: mma.sync fragments for both 16-bit storage types,
// 16-byte gathers, and the score product of one parent's 16 children against the (<= 16) query heads of a group.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "pipe.cuh"

namespace htree {

template <typename T> struct Frag;
template <> struct Frag<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
    static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct Frag<__half> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    }
    static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

// Maximum over the lanes of `members` in one instruction: redux.sync on fp32 is an sm_100a addition.  Use it with the
// full-warp mask: with a different mask per quad it measured several times slower than two shuffles.
__device__ __forceinline__ float redux_max_f32(float x, uint32_t members) {
    float y;
    asm volatile("redux.sync.max.f32 %0, %1, %2;" : "=f"(y) : "f"(x), "r"(members));
    return y;
}
// 2^x, the hardware approximation (what __expf evaluates after its multiply by log2 e)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;

// Packed fp32 arithmetic of sm_100 (two IEEE round-to-nearest operations per instruction): the fp32 query rotation of the
// pass that decides the Top-K is the largest block of scalar work in the selection kernel.
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmul.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rc, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\nfma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
// Half-split rotation of the pair-of-pairs (lo, hi) by (cos, sin): x = lo*cos - hi*sin, y = lo*sin + hi*cos, each as one
// product and one fused multiply-add (nsn = -sin).  One definition for every kernel that rotates in fp32, so that they
// all round alike.
__device__ __forceinline__ void rotate_pairs_f32(float2 lo, float2 hi, float2 cs, float2 sn, float2 nsn, float2& x, float2& y) {
    x = ffma2(hi, nsn, fmul2(lo, cs));
    y = ffma2(hi, cs, fmul2(lo, sn));
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// 32 bytes with one 256-bit load (sm_100a); address must be 32-byte aligned.
__device__ __forceinline__ void ldg32(const void* p, uint32_t (&o)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                 : "l"(p));
}
// The same for gathered rows that are used once: not allocated in L1.  A row that misses L1 otherwise crosses the L1
// data pipe twice (fill, then read), and that pipe is the busiest unit of the attention kernels.
__device__ __forceinline__ void ldg32_stream(const void* p, uint32_t (&o)[8]) {
#ifdef HTREE_LDG_ALLOC
    ldg32(p, o);
#else
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                 : "l"(p));
#endif
}
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
#ifdef HTREE_LDG_ALLOC
    return ldg16(p);
#else
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
#endif
}
// n16 consecutive 16-byte pieces (n16 = 1 or 2) into o[0 .. 4*n16), using one 256-bit load when n16 == 2.
// STREAM: the data is a gathered row (see ldg32_stream).
template <int N16>
__device__ __forceinline__ void ldg_vec(const void* p, bool on, uint32_t* o, bool stream = false) {
    if (N16 == 2) {
        uint32_t t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (on) { if (stream) ldg32_stream(p, t); else ldg32(p, t); }
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = t[i];
    } else {
        uint4 x = make_uint4(0, 0, 0, 0);
        if (on) x = stream ? ldg16_stream(p) : ldg16(p);
        o[0] = x.x; o[1] = x.y; o[2] = x.z; o[3] = x.w;
    }
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Scores of the 16 children of one parent (two n8 tiles: children 0-7 and 8-15) against query rows g and g+8 of the
// group, S = (scale * R(delta) q)^T K'.  Thread (g = lane/4, r = lane%4) owns rotation pairs [PPT*r, PPT*(r+1)) of
// both halves for the contraction (a permutation applied to A and B alike), so keys go from memory to B fragments
// untouched and the query is rotated in registers.  With KEEP_A the rotated-query A fragments of every k-step are
// returned as well (the backward reuses them, transposed, for dK).
//   S0/S1: accumulators of tile 0 / tile 1: [0],[1] = row g, children 2r, 2r+1; [2],[3] = row g+8.
//   qraw holds the query rows as IEEE half pairs (load_rows_half).  ROT16 selects how the query is rotated: false =
//   fp32 arithmetic with the fp32 tables, one rounding to half at the end; true = packed half2 arithmetic with the
//   pre-scaled half tables (4 instead of 14 instructions per pair of pairs, about twice the rounding noise).
//   With KEEP_K (backward) kr receives the keys rotated back into the query's frame, scale * R(-delta) K', in the same
//   fragment order ([tile][half][k-step]); transposed with movmatrix they are the B fragments of dq += dS K~.
//   NR = 1 when the group has at most 8 heads: rows g+8 are padding, their rotation is skipped and their A rows are zero.
//   CR = children per parent (16 or 8).  With 8 the second tile (children 8-15) does not exist: no loads, no MMAs, S1 = 0.
template <int D, bool KEEP_A, bool ROT16, bool KEEP_K = false, int NR = 2, int CR = 16>
__device__ __forceinline__ void score_chunk(const AttnParams& p, const __half* kq, int rstride, int Nl, int node0, int delta,
                                            int g, int r, const uint32_t (&qraw)[2][2][D / 16], float (&S0)[4], float (&S1)[4],
                                            uint32_t (&qa)[KEEP_A ? D / 16 : 1][4], uint32_t (*kr)[2][D / 16] = nullptr, bool stream = true) {
    constexpr int HALF = D / 2, KS = D / 16, PPT = HALF / 4, NV = PPT / 8;
    constexpr bool T1 = CR > 8;   // does tile 1 exist?
    constexpr bool POST_SCALE = !KEEP_A && !KEEP_K && !ROT16;
    using FS = Frag<__half>;
    const float* cp = p.cosc + (size_t)delta * HALF + PPT * r;
    const float* sp = p.sinc + (size_t)delta * HALF + PPT * r;
    // kq = this lane's base into the level (row 0, the group's KV head, column PPT*r; 2*PPT*r for 64-wide rows),
    // rstride = elements per row.
    // Children beyond the end of the level are read from the last row instead: callers mask those columns.
    const int n0 = min(node0 + g, Nl - 1), n1 = min(node0 + 8 + g, Nl - 1);
    const __half* k0 = kq + (int64_t)n0 * rstride;
    const __half* k1 = kq + (int64_t)n1 * rstride;
    uint32_t kb[2][2][KS];   // [tile][half][k-step]
    if (D == 64) {
        // 64-wide rows keep this thread's low and high 8 pairs side by side (rotate_keys_kernel): one 32-byte load per row
        uint32_t t0[8], t1[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        ldg_vec<2>(k0, true, t0, stream);
        if (T1) ldg_vec<2>(k1, true, t1, stream);
#pragma unroll
        for (int i = 0; i < KS; ++i) { kb[0][0][i] = t0[i]; kb[0][1][i] = t0[4 + i]; kb[1][0][i] = t1[i]; kb[1][1][i] = t1[4 + i]; }
    } else {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            ldg_vec<NV>(k0 + hf * HALF, true, kb[0][hf], stream);
            if (T1) ldg_vec<NV>(k1 + hf * HALF, true, kb[1][hf], stream);
            else {
#pragma unroll
                for (int i = 0; i < KS; ++i) kb[1][hf][i] = 0u;
            }
        }
    }
    S0[0] = S0[1] = S0[2] = S0[3] = 0.f;
    S1[0] = S1[1] = S1[2] = S1[3] = 0.f;
    float T0[4] = {0.f, 0.f, 0.f, 0.f}, U1[4] = {0.f, 0.f, 0.f, 0.f};
    if (ROT16) {
        const __half* chp = p.cosh + (size_t)delta * HALF + PPT * r;
        const __half* shp = p.sinh + (size_t)delta * HALF + PPT * r;
        uint32_t ch[KS], sh[KS];   // (cos, sin) * scale of pairs (2ks, 2ks+1), packed half2
        ldg_vec<NV>(chp, true, ch);
        ldg_vec<NV>(shp, true, sh);
        if (KEEP_K) {
#pragma unroll
            for (int tl = 0; tl < (T1 ? 2 : 1); ++tl)
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const __half2 c2 = *reinterpret_cast<const __half2*>(&ch[ks]), s2 = *reinterpret_cast<const __half2*>(&sh[ks]);
                    const __half2 lo = *reinterpret_cast<const __half2*>(&kb[tl][0][ks]), hi = *reinterpret_cast<const __half2*>(&kb[tl][1][ks]);
                    const __half2 u = __hfma2(lo, c2, __hmul2(hi, s2));                 // lo*cos + hi*sin
                    const __half2 w = __hfma2(hi, c2, __hneg2(__hmul2(lo, s2)));        // hi*cos - lo*sin
                    kr[tl][0][ks] = *reinterpret_cast<const uint32_t*>(&u);
                    kr[tl][1][ks] = *reinterpret_cast<const uint32_t*>(&w);
                }
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t a[4];
            const __half2 c2 = *reinterpret_cast<const __half2*>(&ch[ks]), s2 = *reinterpret_cast<const __half2*>(&sh[ks]);
            a[1] = 0u; a[3] = 0u;
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                const __half2 lo = *reinterpret_cast<const __half2*>(&qraw[rr][0][ks]);
                const __half2 hi = *reinterpret_cast<const __half2*>(&qraw[rr][1][ks]);
                const __half2 x = __hfma2(lo, c2, __hneg2(__hmul2(hi, s2)));     // lo*cos - hi*sin
                const __half2 y = __hfma2(hi, c2, __hmul2(lo, s2));              // lo*sin + hi*cos
                a[rr] = *reinterpret_cast<const uint32_t*>(&x);
                a[2 + rr] = *reinterpret_cast<const uint32_t*>(&y);
            }
            if (KEEP_A) { qa[KEEP_A ? ks : 0][0] = a[0]; qa[KEEP_A ? ks : 0][1] = a[1]; qa[KEEP_A ? ks : 0][2] = a[2]; qa[KEEP_A ? ks : 0][3] = a[3]; }
            if (ks & 1) {   // two accumulation chains per tile: halves the dependent-MMA latency on the critical path
                FS::mma(T0, a[0], a[1], a[2], a[3], kb[0][0][ks], kb[0][1][ks]);
                if (T1) FS::mma(U1, a[0], a[1], a[2], a[3], kb[1][0][ks], kb[1][1][ks]);
            } else {
                FS::mma(S0, a[0], a[1], a[2], a[3], kb[0][0][ks], kb[0][1][ks]);
                if (T1) FS::mma(S1, a[0], a[1], a[2], a[3], kb[1][0][ks], kb[1][1][ks]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { S0[i] += T0[i]; S1[i] += U1[i]; }
        if (KEEP_K && !T1) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) { kr[1][0][ks] = 0u; kr[1][1][ks] = 0u; }
        }
        return;
    }
#pragma unroll
    for (int ks2 = 0; ks2 < KS; ks2 += 2) {
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(cp + 2 * ks2));
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(sp + 2 * ks2));
        // the softmax scale goes into the tables, or, when only the scores are wanted, onto the 8 scores at the end
        const float tsc = POST_SCALE ? 1.f : p.scale;
        const float cs[4] = {c4.x * tsc, c4.y * tsc, c4.z * tsc, c4.w * tsc};
        const float sn[4] = {s4.x * tsc, s4.y * tsc, s4.z * tsc, s4.w * tsc};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int ks = ks2 + u;
            uint32_t a[4];
            a[1] = 0u; a[3] = 0u;
#pragma unroll
            const float2 c2 = make_float2(cs[2 * u], cs[2 * u + 1]), s2 = make_float2(sn[2 * u], sn[2 * u + 1]);
            const float2 ns2 = make_float2(-s2.x, -s2.y);
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                float2 x, y;
                rotate_pairs_f32(FS::unpack(qraw[rr][0][ks]), FS::unpack(qraw[rr][1][ks]), c2, s2, ns2, x, y);
                a[rr] = FS::pack(x.x, x.y);         // rotated low half
                a[2 + rr] = FS::pack(y.x, y.y);     // rotated high half
            }
            if (KEEP_A) { qa[KEEP_A ? ks : 0][0] = a[0]; qa[KEEP_A ? ks : 0][1] = a[1]; qa[KEEP_A ? ks : 0][2] = a[2]; qa[KEEP_A ? ks : 0][3] = a[3]; }
            if (KEEP_K) {
#pragma unroll
                for (int tl = 0; tl < 2; ++tl) {
                    if (!T1 && tl == 1) { kr[1][0][ks] = 0u; kr[1][1][ks] = 0u; continue; }
                    const float2 lo = FS::unpack(kb[tl][0][ks]), hi = FS::unpack(kb[tl][1][ks]);
                    const float c0 = cs[2 * u], c1 = cs[2 * u + 1], s0 = sn[2 * u], s1 = sn[2 * u + 1];
                    kr[tl][0][ks] = FS::pack(lo.x * c0 + hi.x * s0, lo.y * c1 + hi.y * s1);
                    kr[tl][1][ks] = FS::pack(hi.x * c0 - lo.x * s0, hi.y * c1 - lo.y * s1);
                }
            }
            if (u) {
                FS::mma(T0, a[0], a[1], a[2], a[3], kb[0][0][ks], kb[0][1][ks]);
                if (T1) FS::mma(U1, a[0], a[1], a[2], a[3], kb[1][0][ks], kb[1][1][ks]);
            } else {
                FS::mma(S0, a[0], a[1], a[2], a[3], kb[0][0][ks], kb[0][1][ks]);
                if (T1) FS::mma(S1, a[0], a[1], a[2], a[3], kb[1][0][ks], kb[1][1][ks]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        S0[i] += T0[i]; S1[i] += U1[i];
        if (POST_SCALE) { S0[i] *= p.scale; S1[i] *= p.scale; }
    }
}

// score_chunk with the key fragments read from shared memory: `ks4` is a parent's blocked keys in fragment-major order
// (tree.cu: piece [ks][lane] = the four B-fragment registers of k-step ks), so each 16-byte shared load feeds the two
// MMAs of one k-step.  Same arithmetic, operand values and accumulation order as score_chunk.
template <int D, bool ROT16, int NR>
__device__ __forceinline__ void score_chunk_sm(const AttnParams& p, const uint4* ks4, const unsigned char* tab, int lane,
                                               const uint32_t (&qraw)[2][2][D / 16], float (&S0)[4], float (&S1)[4]) {
    // tab: the chunk's table rows in shared memory: ROT16 ? [cos*scale | sin*scale] as IEEE half (D/2 each)
    //                                                      : [cos | sin] as fp32 (D/2 each)
    constexpr int HALF = D / 2, KS = D / 16, PPT = HALF / 4;
    using FS = Frag<__half>;
    const int r = lane & 3;
    S0[0] = S0[1] = S0[2] = S0[3] = 0.f;
    S1[0] = S1[1] = S1[2] = S1[3] = 0.f;
    float T0[4] = {0.f, 0.f, 0.f, 0.f}, U1[4] = {0.f, 0.f, 0.f, 0.f};
    if (ROT16) {
        uint32_t ch[KS], sh[KS];   // (cos, sin) * scale of pairs (2ks, 2ks+1), packed half2: this lane's PPT pairs
#pragma unroll
        for (int i = 0; i < KS / 4; ++i) {
            const uint4 c4 = lds128(tab + 2 * (PPT * r) + 16 * i);
            const uint4 s4 = lds128(tab + 2 * HALF + 2 * (PPT * r) + 16 * i);
            ch[4 * i] = c4.x; ch[4 * i + 1] = c4.y; ch[4 * i + 2] = c4.z; ch[4 * i + 3] = c4.w;
            sh[4 * i] = s4.x; sh[4 * i + 1] = s4.y; sh[4 * i + 2] = s4.z; sh[4 * i + 3] = s4.w;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint4 kb = lds128(ks4 + ks * 32 + lane);
            uint32_t a[4];
            const __half2 c2 = *reinterpret_cast<const __half2*>(&ch[ks]), s2 = *reinterpret_cast<const __half2*>(&sh[ks]);
            a[1] = 0u; a[3] = 0u;
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                const __half2 lo = *reinterpret_cast<const __half2*>(&qraw[rr][0][ks]);
                const __half2 hi = *reinterpret_cast<const __half2*>(&qraw[rr][1][ks]);
                const __half2 x = __hfma2(lo, c2, __hneg2(__hmul2(hi, s2)));
                const __half2 y = __hfma2(hi, c2, __hmul2(lo, s2));
                a[rr] = *reinterpret_cast<const uint32_t*>(&x);
                a[2 + rr] = *reinterpret_cast<const uint32_t*>(&y);
            }
            if (ks & 1) {
                FS::mma(T0, a[0], a[1], a[2], a[3], kb.x, kb.y);
                FS::mma(U1, a[0], a[1], a[2], a[3], kb.z, kb.w);
            } else {
                FS::mma(S0, a[0], a[1], a[2], a[3], kb.x, kb.y);
                FS::mma(S1, a[0], a[1], a[2], a[3], kb.z, kb.w);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { S0[i] += T0[i]; S1[i] += U1[i]; }
        return;
    }
    const unsigned char* cp = tab + 4 * (PPT * r);
    const unsigned char* sp = tab + 4 * HALF + 4 * (PPT * r);
#pragma unroll
    for (int ks2 = 0; ks2 < KS; ks2 += 2) {
        const uint4 c4 = lds128(cp + 8 * ks2);
        const uint4 s4 = lds128(sp + 8 * ks2);
        const float cs[4] = {__uint_as_float(c4.x), __uint_as_float(c4.y), __uint_as_float(c4.z), __uint_as_float(c4.w)};
        const float sn[4] = {__uint_as_float(s4.x), __uint_as_float(s4.y), __uint_as_float(s4.z), __uint_as_float(s4.w)};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int ks = ks2 + u;
            const uint4 kb = lds128(ks4 + ks * 32 + lane);
            uint32_t a[4];
            a[1] = 0u; a[3] = 0u;
#pragma unroll
            const float2 c2 = make_float2(cs[2 * u], cs[2 * u + 1]), s2 = make_float2(sn[2 * u], sn[2 * u + 1]);
            const float2 ns2 = make_float2(-s2.x, -s2.y);
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                float2 x, y;
                rotate_pairs_f32(FS::unpack(qraw[rr][0][ks]), FS::unpack(qraw[rr][1][ks]), c2, s2, ns2, x, y);
                a[rr] = FS::pack(x.x, x.y);
                a[2 + rr] = FS::pack(y.x, y.y);
            }
            if (u) {
                FS::mma(T0, a[0], a[1], a[2], a[3], kb.x, kb.y);
                FS::mma(U1, a[0], a[1], a[2], a[3], kb.z, kb.w);
            } else {
                FS::mma(S0, a[0], a[1], a[2], a[3], kb.x, kb.y);
                FS::mma(S1, a[0], a[1], a[2], a[3], kb.z, kb.w);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { S0[i] = (S0[i] + T0[i]) * p.scale; S1[i] = (S1[i] + U1[i]) * p.scale; }
}

// Raw rows g and g+8 of a [heads, D] block in the fragment order used above (zero for rows beyond the group).
template <typename T, int D>
__device__ __forceinline__ void load_rows(const T* base, int g, int r, const bool (&row_ok)[2], uint32_t (&raw)[2][2][D / 16]) {
    constexpr int HALF = D / 2, PPT = HALF / 4, NV = PPT / 8;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const T* row = base + (int64_t)(g + 8 * rr) * D;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) ldg_vec<NV>(row + hf * HALF + PPT * r, row_ok[rr], raw[rr][hf]);
    }
}

// Query rows for score_chunk: load_rows, then bf16 pairs are converted to IEEE half pairs (exact for magnitudes in
// half's normal range; larger values saturate to the largest finite half).
template <typename T, int D>
__device__ __forceinline__ void load_rows_half(const T* base, int g, int r, const bool (&row_ok)[2], uint32_t (&raw)[2][2][D / 16]) {
    load_rows<T, D>(base, g, r, row_ok, raw);
    if (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                for (int i = 0; i < D / 16; ++i) {
                    const float2 f = Frag<__nv_bfloat16>::unpack(raw[rr][hf][i]);
                    raw[rr][hf][i] = Frag<__half>::pack(fminf(fmaxf(f.x, -65504.f), 65504.f), fminf(fmaxf(f.y, -65504.f), 65504.f));
                }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// fp32 storage on the tensor cores: split-half products.  A value x is carried as hi = half(x) and lo = half(x - hi)
// (22 significand bits together); a product of two such values is formed as hi*hi + hi*lo + lo*hi by three
// mma.sync.m16n8k16 f16 instructions with fp32 accumulation (lo*lo is below fp32 resolution).  This keeps the scores,
// and with them the Top-K decisions, at fp32 accuracy, which single TF32 / half products (10-11 bits) do not.
// 64-wide heads only: the fp32 query rows already take 32 registers per thread.

// two floats -> packed (hi, hi) and (lo, lo) half pairs
__device__ __forceinline__ void split_half2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 f = __half22float2(h);
    const __half2 l = __floats2half2_rn(x0 - f.x, x1 - f.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// fp32 rows g and g+8 of a [heads, D] block: raw[rr][hf][i] = bits of element hf*D/2 + PPT*r + i (zero for rows beyond the group)
template <int D>
__device__ __forceinline__ void load_rows_f32(const float* base, int g, int r, const bool (&row_ok)[2], uint32_t (&raw)[2][2][D / 8]) {
    constexpr int HALF = D / 2, PPT = HALF / 4;
    static_assert(PPT == 8, "split-half kernels are built for 64-wide heads");
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) ldg_vec<2>(base + (int64_t)(g + 8 * rr) * D + hf * HALF + PPT * r, row_ok[rr], raw[rr][hf]);
}

// score_chunk for fp32 storage, D = 64.  kq points at this lane's piece of the hi plane of K' (plane elements further: the
// lo plane); qf holds the fp32 query rows (load_rows_f32).  The query is rotated and scaled in fp32, then split.
// With KEEP (backward) the rotated-query fragments (qa_hi/qa_lo [ks][4]) and the keys rotated back into the query's
// frame (fp32, kr[tile][half][2*ks + {0,1}]) are returned as well.
template <int D, int NR, int CR, bool KEEP = false>
__device__ __forceinline__ void score_chunk_x3(const AttnParams& p, const __half* kq, int64_t plane, int rstride, int Nl, int node0,
                                               int delta, int g, int r, const uint32_t (&qf)[2][2][D / 8], float (&S0)[4],
                                               float (&S1)[4], bool stream, uint32_t (*qa_hi)[4] = nullptr,
                                               uint32_t (*qa_lo)[4] = nullptr, float (*kr)[2][D / 8] = nullptr) {
    constexpr int HALF = D / 2, KS = D / 16, PPT = HALF / 4;
    constexpr bool T1 = CR > 8;
    using FS = Frag<__half>;
    const int n0 = min(node0 + g, Nl - 1), n1 = min(node0 + 8 + g, Nl - 1);
    uint32_t kh[2][2][KS], kl[2][2][KS];   // [tile][half][k-step], hi and lo planes
    {
        uint32_t t0[8], t1[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u}, u0[8], u1[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        const __half* k0 = kq + (int64_t)n0 * rstride;
        const __half* k1 = kq + (int64_t)n1 * rstride;
        ldg_vec<2>(k0, true, t0, stream); ldg_vec<2>(k0 + plane, true, u0, stream);
        if (T1) { ldg_vec<2>(k1, true, t1, stream); ldg_vec<2>(k1 + plane, true, u1, stream); }
#pragma unroll
        for (int i = 0; i < KS; ++i) {
            kh[0][0][i] = t0[i]; kh[0][1][i] = t0[4 + i]; kh[1][0][i] = t1[i]; kh[1][1][i] = t1[4 + i];
            kl[0][0][i] = u0[i]; kl[0][1][i] = u0[4 + i]; kl[1][0][i] = u1[i]; kl[1][1][i] = u1[4 + i];
        }
    }
    float cs[PPT], sn[PPT];
    {
        const float4* cp = reinterpret_cast<const float4*>(p.cosc + (size_t)delta * HALF + PPT * r);
        const float4* sp = reinterpret_cast<const float4*>(p.sinc + (size_t)delta * HALF + PPT * r);
#pragma unroll
        for (int i = 0; i < PPT / 4; ++i) {
            const float4 c4 = __ldg(cp + i), s4 = __ldg(sp + i);
            cs[4 * i] = c4.x * p.scale; cs[4 * i + 1] = c4.y * p.scale; cs[4 * i + 2] = c4.z * p.scale; cs[4 * i + 3] = c4.w * p.scale;
            sn[4 * i] = s4.x * p.scale; sn[4 * i + 1] = s4.y * p.scale; sn[4 * i + 2] = s4.z * p.scale; sn[4 * i + 3] = s4.w * p.scale;
        }
    }
    float A0[4] = {0.f, 0.f, 0.f, 0.f}, B0[4] = {0.f, 0.f, 0.f, 0.f}, C0[4] = {0.f, 0.f, 0.f, 0.f};
    float A1[4] = {0.f, 0.f, 0.f, 0.f}, B1[4] = {0.f, 0.f, 0.f, 0.f}, C1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        uint32_t ah[4] = {0u, 0u, 0u, 0u}, al[4] = {0u, 0u, 0u, 0u};
        const float c0 = cs[2 * ks], c1 = cs[2 * ks + 1], s0 = sn[2 * ks], s1 = sn[2 * ks + 1];
        const float2 c2 = make_float2(c0, c1), s2 = make_float2(s0, s1), ns2 = make_float2(-s0, -s1);
#pragma unroll
        for (int rr = 0; rr < NR; ++rr) {
            const float2 lo = make_float2(__uint_as_float(qf[rr][0][2 * ks]), __uint_as_float(qf[rr][0][2 * ks + 1]));
            const float2 hi = make_float2(__uint_as_float(qf[rr][1][2 * ks]), __uint_as_float(qf[rr][1][2 * ks + 1]));
            float2 x, y;
            rotate_pairs_f32(lo, hi, c2, s2, ns2, x, y);
            split_half2(x.x, x.y, ah[rr], al[rr]);              // rotated low half
            split_half2(y.x, y.y, ah[2 + rr], al[2 + rr]);      // rotated high half
        }
        if (KEEP) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { qa_hi[ks][i] = ah[i]; qa_lo[ks][i] = al[i]; }
#pragma unroll
            for (int tl = 0; tl < 2; ++tl) {
                if (!T1 && tl == 1) { kr[1][0][2 * ks] = kr[1][0][2 * ks + 1] = kr[1][1][2 * ks] = kr[1][1][2 * ks + 1] = 0.f; continue; }
                const float2 lh = FS::unpack(kh[tl][0][ks]), ll = FS::unpack(kl[tl][0][ks]);
                const float2 hh = FS::unpack(kh[tl][1][ks]), hl = FS::unpack(kl[tl][1][ks]);
                const float klx = lh.x + ll.x, kly = lh.y + ll.y, khx = hh.x + hl.x, khy = hh.y + hl.y;
                kr[tl][0][2 * ks] = klx * c0 + khx * s0; kr[tl][0][2 * ks + 1] = kly * c1 + khy * s1;      // scale * R(-delta) K'
                kr[tl][1][2 * ks] = khx * c0 - klx * s0; kr[tl][1][2 * ks + 1] = khy * c1 - kly * s1;
            }
        }
        // The hi*hi product of every k-step starts from a zero accumulator and is added to the running sum with an ordinary
        // (round-to-nearest) fp32 add: inside the MMA the 16 products and the accumulator are aligned to the largest of
        // them and truncated, so a running score of magnitude 2^6 in the accumulator would cost 8x the rounding error of
        // the products alone, and always in the same direction.  The hi*lo chains are 2^-11 smaller: no such concern.
        float h0[4] = {0.f, 0.f, 0.f, 0.f}, h1[4] = {0.f, 0.f, 0.f, 0.f};
        FS::mma(h0, ah[0], ah[1], ah[2], ah[3], kh[0][0][ks], kh[0][1][ks]);
        FS::mma(B0, ah[0], ah[1], ah[2], ah[3], kl[0][0][ks], kl[0][1][ks]);
        FS::mma(C0, al[0], al[1], al[2], al[3], kh[0][0][ks], kh[0][1][ks]);
        if (T1) {
            FS::mma(h1, ah[0], ah[1], ah[2], ah[3], kh[1][0][ks], kh[1][1][ks]);
            FS::mma(B1, ah[0], ah[1], ah[2], ah[3], kl[1][0][ks], kl[1][1][ks]);
            FS::mma(C1, al[0], al[1], al[2], al[3], kh[1][0][ks], kh[1][1][ks]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { A0[i] += h0[i]; A1[i] += h1[i]; }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { S0[i] = A0[i] + (B0[i] + C0[i]); S1[i] = A1[i] + (B1[i] + C1[i]); }
}

}  // namespace htree
