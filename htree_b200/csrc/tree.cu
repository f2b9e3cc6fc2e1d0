// Mean-pool tree build and its gradient: HBM-streaming kernels.
//
// A level is stored [B, N, H_kv, D]; a parent row (all KV heads, W = H_kv*D elements) is the mean of the CR child
// rows below it, which lie contiguously in memory, so one thread owns one 16-byte column of a parent row and walks
// its children with independent 128-bit loads.  Reference behaviour: htree_build_kernel (src/parallel.py:87-181)
// and htree_bwd_tree_backward_kernel (src/backward.py:787-841); numerics follow src/naive.py:53-57 (fp32 sum,
// division by the number of valid children, one rounding to the storage type).
#include "common.cuh"

namespace htree {

template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec16<__half> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void unpack16(const uint4& r, float* o);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& r, float* o) {
    o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y); o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& r, float* o) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& r, float* o) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float* o);
template <> __device__ __forceinline__ uint4 pack16<float>(const float* o) {
    return make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3]));
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float* o) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack16<__half>(const float* o) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

struct BuildArgs {
    const void* child[2];
    void* parent[2];
    int32_t wv[2];      // 16-byte vectors per row (row = all KV heads of one node)
    int64_t total[2];   // B * Np * wv
    int32_t Nc, Np, CR;
};

// blockIdx.y = 0 pools K, 1 pools V.  UNR = children loaded per unrolled batch.
template <typename T, int UNR>
__global__ void __launch_bounds__(256) tree_build_kernel(const __grid_constant__ BuildArgs a) {
    constexpr int VN = Vec16<T>::N;
    const int which = blockIdx.y;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total[which]) return;
    const int wv = a.wv[which];
    const int col = (int)(idx % wv);
    const int64_t row = idx / wv;            // b * Np + p
    const int p = (int)(row % a.Np);
    const int64_t b = row / a.Np;
    const int first = p * a.CR;
    const int cnt = min(a.CR, a.Nc - first);
    const uint4* src = reinterpret_cast<const uint4*>(a.child[which]) + ((b * a.Nc + first) * (int64_t)wv + col);
    float acc[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] = 0.f;
    for (int c0 = 0; c0 < cnt; c0 += UNR) {
        uint4 r[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u)
            if (c0 + u < cnt) r[u] = __ldcs(src + (int64_t)(c0 + u) * wv);   // streamed once: evict-first
#pragma unroll
        for (int u = 0; u < UNR; ++u)
            if (c0 + u < cnt) {
                float f[VN];
                unpack16<T>(r[u], f);
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[i] += f[i];
            }
    }
    const float n = (float)cnt;
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] = acc[i] / n;
    reinterpret_cast<uint4*>(a.parent[which])[row * wv + col] = pack16<T>(acc);
}

template <typename T>
static int build_levels(const HtreeShape& s, int L, const int32_t* ln, void* const* lk, void* const* lv, cudaStream_t st) {
    constexpr int VN = Vec16<T>::N;
    for (int l = 1; l < L; ++l) {
        BuildArgs a;
        a.child[0] = lk[l - 1]; a.child[1] = lv[l - 1];
        a.parent[0] = lk[l]; a.parent[1] = lv[l];
        a.wv[0] = s.H_kv * s.K / VN; a.wv[1] = s.H_kv * s.V / VN;
        a.Nc = ln[l - 1]; a.Np = ln[l]; a.CR = s.compression_rate;
        a.total[0] = (int64_t)s.B * a.Np * a.wv[0]; a.total[1] = (int64_t)s.B * a.Np * a.wv[1];
        int64_t mx = a.total[0] > a.total[1] ? a.total[0] : a.total[1];
        dim3 grid((unsigned)((mx + 255) / 256), 2);
#ifndef HTREE_BUILD_UNR
#define HTREE_BUILD_UNR 8   // children loaded per batch: 8 keeps 80 registers and 3 blocks per SM (82 % of HBM peak vs 51 % with 16)
#endif
        if (s.compression_rate >= 16) tree_build_kernel<T, HTREE_BUILD_UNR><<<grid, 256, 0, st>>>(a);
        else tree_build_kernel<T, 8><<<grid, 256, 0, st>>>(a);
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

int launch_tree_build(const HtreeShape& s, int L, const int32_t* ln, void* const* lk, void* const* lv, cudaStream_t st) {
    switch (s.dtype) {
        case HTREE_F32: return build_levels<float>(s, L, ln, lk, lv, st);
        case HTREE_BF16: return build_levels<__nv_bfloat16>(s, L, ln, lk, lv, st);
        default: return build_levels<__half>(s, L, ln, lk, lv, st);
    }
}

struct RotArgs {
    const void* src;
    void* dst;
    const float* cosc;
    const float* sinc;
    int64_t total;     // rows * (K/16): one thread rotates 8 pairs
    int64_t plane;     // fp32 storage only: elements between the hi plane and the lo plane of the destination
    int32_t Hkv, K, N, CR;
};

// K'[b, node, h, :] = R(node % CR) K[b, node, h, :] (half-split rotation by the child index), 16-bit storage types.
// The tensor-core attention kernels read K' so that the per-candidate rotation of the reference
// (src/parallel.py:687-692) turns into one query rotation per parent.
// K' is always written as IEEE half, also for bf16 inputs: the rotated value is not representable in either type, and
// half's 11-bit significand makes the one rounding 8x smaller than bf16's would be, which is what decides how often
// Top-K boundary nodes swap against an fp32 evaluation.  Values are clamped to the finite half range.
template <typename T>
__global__ void __launch_bounds__(256) rotate_keys_kernel(const __grid_constant__ RotArgs a) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int half = a.K >> 1, cpr = half >> 3;          // 8-pair chunks per row
    const int ch = (int)(idx % cpr);
    const int64_t row = idx / cpr;                        // (b * N + node) * Hkv + h
    const int node = (int)((row / a.Hkv) % a.N);
    const int c = node % a.CR;
    const T* src = reinterpret_cast<const T*>(a.src) + row * a.K + 8 * ch;
    __half* dst = reinterpret_cast<__half*>(a.dst) + row * a.K + 8 * ch;
    float lo[8], hi[8], cs[8], sn[8];
    unpack16<T>(__ldg(reinterpret_cast<const uint4*>(src)), lo);
    unpack16<T>(__ldg(reinterpret_cast<const uint4*>(src + half)), hi);
    const float4* cp = reinterpret_cast<const float4*>(a.cosc + (int64_t)c * half + 8 * ch);
    const float4* sp = reinterpret_cast<const float4*>(a.sinc + (int64_t)c * half + 8 * ch);
    const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
    cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    float olo[8], ohi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        olo[i] = fminf(fmaxf(lo[i] * cs[i] - hi[i] * sn[i], -65504.f), 65504.f);
        ohi[i] = fminf(fmaxf(lo[i] * sn[i] + hi[i] * cs[i], -65504.f), 65504.f);
    }
    if (a.K == 64) {
        // 64-wide rows: the low and the high 8 pairs that one thread of the tensor-core kernels owns are stored side by
        // side (chunk ch at [16 ch, 16 ch + 16)), so that it fetches both with a single 32-byte load
        __half* row0 = reinterpret_cast<__half*>(a.dst) + row * a.K;
        *reinterpret_cast<uint4*>(row0 + 16 * ch) = pack16<__half>(olo);
        *reinterpret_cast<uint4*>(row0 + 16 * ch + 8) = pack16<__half>(ohi);
    } else {
        *reinterpret_cast<uint4*>(dst) = pack16<__half>(olo);
        *reinterpret_cast<uint4*>(dst + half) = pack16<__half>(ohi);
    }
}

// fp32 storage, 64-wide rows: K' = R(node % CR) K in fp32, written as TWO IEEE-half planes hi = half(K'), lo = half(K' - hi)
// (plane 1 follows plane 0, each shaped and ordered like the 16-bit K' of 64-wide rows).  hi + lo carries 22 significand
// bits; the split-half tensor-core kernels form q.k as q_hi.k_hi + q_hi.k_lo + q_lo.k_hi with fp32 accumulation.
__global__ void __launch_bounds__(256) rotate_keys_split_kernel(const __grid_constant__ RotArgs a) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int half = a.K >> 1, cpr = half >> 3;
    const int ch = (int)(idx % cpr);
    const int64_t row = idx / cpr;
    const int node = (int)((row / a.Hkv) % a.N);
    const int c = node % a.CR;
    const float* src = reinterpret_cast<const float*>(a.src) + row * a.K + 8 * ch;
    float lo[8], hi[8], cs[8], sn[8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(src) + i), y = __ldg(reinterpret_cast<const float4*>(src + half) + i);
        lo[4 * i] = x.x; lo[4 * i + 1] = x.y; lo[4 * i + 2] = x.z; lo[4 * i + 3] = x.w;
        hi[4 * i] = y.x; hi[4 * i + 1] = y.y; hi[4 * i + 2] = y.z; hi[4 * i + 3] = y.w;
        const float4 cc = __ldg(reinterpret_cast<const float4*>(a.cosc + (int64_t)c * half + 8 * ch) + i);
        const float4 ss = __ldg(reinterpret_cast<const float4*>(a.sinc + (int64_t)c * half + 8 * ch) + i);
        cs[4 * i] = cc.x; cs[4 * i + 1] = cc.y; cs[4 * i + 2] = cc.z; cs[4 * i + 3] = cc.w;
        sn[4 * i] = ss.x; sn[4 * i + 1] = ss.y; sn[4 * i + 2] = ss.z; sn[4 * i + 3] = ss.w;
    }
    float olo[8], ohi[8], rlo[8], rhi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x = fminf(fmaxf(lo[i] * cs[i] - hi[i] * sn[i], -65504.f), 65504.f);
        const float y = fminf(fmaxf(lo[i] * sn[i] + hi[i] * cs[i], -65504.f), 65504.f);
        olo[i] = __half2float(__float2half_rn(x)); rlo[i] = x - olo[i];
        ohi[i] = __half2float(__float2half_rn(y)); rhi[i] = y - ohi[i];
    }
    // 64-wide rows: chunk ch holds its 8 low pairs then its 8 high pairs (see rotate_keys_kernel)
    __half* p0 = reinterpret_cast<__half*>(a.dst) + row * a.K + 16 * ch;
    __half* p1 = p0 + a.plane;
    *reinterpret_cast<uint4*>(p0) = pack16<__half>(olo); *reinterpret_cast<uint4*>(p0 + 8) = pack16<__half>(ohi);
    *reinterpret_cast<uint4*>(p1) = pack16<__half>(rlo); *reinterpret_cast<uint4*>(p1 + 8) = pack16<__half>(rhi);
}

int launch_rotate_keys(const HtreeShape& s, int L, const int32_t* ln, void* const* lk, void* const* lkr, const float* cosc,
                       const float* sinc, cudaStream_t st) {
    if ((s.K % 16) != 0 || (s.dtype == HTREE_F32 && s.K != 64)) return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L; ++l) {
        RotArgs a;
        a.src = lk[l]; a.dst = lkr[l]; a.cosc = cosc; a.sinc = sinc;
        a.Hkv = s.H_kv; a.K = s.K; a.N = ln[l]; a.CR = s.compression_rate;
        a.total = (int64_t)s.B * ln[l] * s.H_kv * (s.K / 16);
        a.plane = (int64_t)s.B * ln[l] * s.H_kv * s.K;
        const unsigned grid = (unsigned)((a.total + 255) / 256);
        if (s.dtype == HTREE_F32) rotate_keys_split_kernel<<<grid, 256, 0, st>>>(a);
        else if (s.dtype == HTREE_BF16) rotate_keys_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
        else rotate_keys_kernel<__half><<<grid, 256, 0, st>>>(a);
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

struct BlkArgs {
    const void* src;
    void* dst;
    int64_t total;     // B * NBLK * Hkv * 32: one thread writes the piece one lane of the attention kernels reads
    int64_t plane;     // fp32 storage only: elements between the hi plane and the lo plane of the destination
    int32_t Hkv, N, NBLK;
};

// V^ ("blocked values"): the rows of one parent's CR children, re-laid-out so that every lane of a warp of the
// tensor-core forward fetches the B fragments of its P.V products (mma.sync.m16n8k16, k = child, n = value column) as one
// contiguous piece, with no byte permutes and fully coalesced (the warp reads the block's CR*D*2 bytes front to back).
// Block (b, p, h) starts at ((b*NBLK + p)*Hkv + h) * CR*D elements; inside it, lane (g = lane/4... see below) owns
//   word ((r*8 + g)*NOT + w)*NB + j  =  { V[p*CR + 8j + 2r][VB*g + w],  V[p*CR + 8j + 2r + 1][VB*g + w] }
// with r = 0..3, g = 0..7, w = 0..NOT-1 (NOT = VB = D/8 output tiles), j = 0..NB-1 (NB = CR/8 registers per tile).
// Rows beyond the end of the level are zero.  16-bit storage types; the values are copied bit for bit.
// SPLIT (fp32 storage): the source rows are fp32 and two planes are written, hi = half(v) and lo = half(v - hi).
template <int D, int CR, bool SPLIT>
__global__ void __launch_bounds__(256) block_values_kernel(const __grid_constant__ BlkArgs a) {
    constexpr int NOT = D / 8, NB = CR / 8, CHW = NOT * NB;     // CHW 32-bit words per lane
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int slot = (int)(idx & 31), r = slot >> 3, g = slot & 7;
    const int64_t blk = idx >> 5;                      // (b * NBLK + p) * Hkv + h
    const int h = (int)(blk % a.Hkv);
    const int p = (int)((blk / a.Hkv) % a.NBLK);
    const int64_t b = blk / ((int64_t)a.Hkv * a.NBLK);
    uint16_t e[NB][2][NOT], elo[SPLIT ? NB : 1][2][NOT];
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int row = p * CR + 8 * j + 2 * r + u;
            const bool ok = row < a.N;
            const int64_t off = ((b * a.N + (ok ? row : 0)) * a.Hkv + h) * (int64_t)D + NOT * g;
            if (SPLIT) {
                const float4* rp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.src) + off);
#pragma unroll
                for (int i = 0; i < NOT / 4; ++i) {
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (ok) x = __ldg(rp + i);
                    const float f4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float v = fminf(fmaxf(f4[q], -65504.f), 65504.f);
                        const __half hv = __float2half_rn(v);
                        const __half lv = __float2half_rn(v - __half2float(hv));
                        e[j][u][4 * i + q] = __half_as_ushort(hv);
                        elo[SPLIT ? j : 0][u][4 * i + q] = __half_as_ushort(lv);
                    }
                }
            } else {
                const uint4* rp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.src) + off);
#pragma unroll
                for (int i = 0; i < NOT / 8; ++i) {
                    uint4 x = make_uint4(0u, 0u, 0u, 0u);
                    if (ok) x = __ldg(rp + i);
                    const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) { e[j][u][8 * i + 2 * q] = (uint16_t)(w4[q] & 0xffffu); e[j][u][8 * i + 2 * q + 1] = (uint16_t)(w4[q] >> 16); }
                }
            }
        }
    if (kFragmentMajor<D, CR, SPLIT>) {
        // fragment-major order (128-wide heads, 16 children, 16-bit types): 16-byte piece i of lane (g, r) sits at
        // [i][4g + r], so that a warp reading piece i from shared memory touches 512 consecutive bytes, and piece i is
        // exactly what output tiles 2i and 2i+1 need: {b0(2i), b1(2i), b0(2i+1), b1(2i+1)}
        uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(a.dst) + blk * (int64_t)(CR * D / 2));
        const int lane = 4 * g + r;
#pragma unroll
        for (int i = 0; i < CHW / 4; ++i) {
            uint32_t o4[4];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int j = 0; j < NB; ++j) o4[u * NB + j] = (uint32_t)e[j][0][2 * i + u] | ((uint32_t)e[j][1][2 * i + u] << 16);
            d4[i * 32 + lane] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
        return;
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(a.dst) + blk * (int64_t)(CR * D / 2) + (int64_t)slot * CHW;
#pragma unroll
    for (int pl = 0; pl < (SPLIT ? 2 : 1); ++pl) {
        uint32_t o[CHW];
#pragma unroll
        for (int w = 0; w < NOT; ++w)
#pragma unroll
            for (int j = 0; j < NB; ++j)
                o[w * NB + j] = pl == 0 ? ((uint32_t)e[j][0][w] | ((uint32_t)e[j][1][w] << 16))
                                        : ((uint32_t)elo[SPLIT ? j : 0][0][w] | ((uint32_t)elo[SPLIT ? j : 0][1][w] << 16));
        uint32_t* d = dst + (pl ? a.plane / 2 : 0);
#pragma unroll
        for (int i = 0; i < CHW / 4; ++i) reinterpret_cast<uint4*>(d)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
    }
}

// K'^ ("blocked keys", 128-wide heads, 16 children, 16-bit types): the pre-rotated key rows of one parent's children in
// fragment-major order.  Block (b, p, h) starts at ((b*NBLK + p)*Hkv + h) * 16*128 halves; its 16-byte piece [ks][4g + r]
// holds, for k-step ks of the score product, the four B-fragment registers of lane (g, r):
//   { K'[16p + g][16r + 2ks, +1],  K'[16p + g][64 + 16r + 2ks, +1],  K'[16p + 8 + g][16r + 2ks, +1],  K'[16p + 8 + g][64 + 16r + 2ks, +1] }
// (tile 0 low half, tile 0 high half, tile 1 low half, tile 1 high half).  Rows past the end of the level are zero.
__global__ void __launch_bounds__(256) block_keys_kernel(const __grid_constant__ BlkArgs a) {
    constexpr int D = 128, CR = 16, KS = 8;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int lane = (int)(idx & 31), g = lane >> 2, r = lane & 3;
    const int64_t blk = idx >> 5;
    const int h = (int)(blk % a.Hkv);
    const int p = (int)((blk / a.Hkv) % a.NBLK);
    const int64_t b = blk / ((int64_t)a.Hkv * a.NBLK);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.src);      // half pairs
    uint32_t kb[2][2][KS];
#pragma unroll
    for (int tl = 0; tl < 2; ++tl) {
        const int row = p * CR + 8 * tl + g;
        const bool ok = row < a.N;
        const int64_t off = (((b * a.N + (ok ? row : 0)) * a.Hkv + h) * (int64_t)D + 16 * r) / 2;   // in 32-bit words
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint4 x = make_uint4(0u, 0u, 0u, 0u);
                if (ok) x = __ldg(reinterpret_cast<const uint4*>(src + off + hf * (D / 4)) + i);
                kb[tl][hf][4 * i] = x.x; kb[tl][hf][4 * i + 1] = x.y; kb[tl][hf][4 * i + 2] = x.z; kb[tl][hf][4 * i + 3] = x.w;
            }
    }
    uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(a.dst) + blk * (int64_t)(CR * D / 2));
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) d4[ks * 32 + lane] = make_uint4(kb[0][0][ks], kb[0][1][ks], kb[1][0][ks], kb[1][1][ks]);
}

int launch_block_keys(const HtreeShape& s, int L, const int32_t* ln, void* const* lkr, void* const* lkb, cudaStream_t st) {
    if (s.dtype == HTREE_F32 || s.K != 128 || s.compression_rate != 16) return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L; ++l) {
        BlkArgs a;
        a.src = lkr[l]; a.dst = lkb[l];
        a.Hkv = s.H_kv; a.N = ln[l]; a.NBLK = (ln[l] + 15) / 16;
        a.total = (int64_t)s.B * a.NBLK * s.H_kv * 32;
        a.plane = 0;
        block_keys_kernel<<<(unsigned)((a.total + 255) / 256), 256, 0, st>>>(a);
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

int launch_block_values(const HtreeShape& s, int L, const int32_t* ln, void* const* lv, void* const* lvb, cudaStream_t st) {
    const int CR = s.compression_rate, D = s.V;
    if ((D != 64 && D != 128) || (CR != 8 && CR != 16) || (s.dtype == HTREE_F32 && D != 64)) return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L; ++l) {
        BlkArgs a;
        a.src = lv[l]; a.dst = lvb[l];
        a.Hkv = s.H_kv; a.N = ln[l]; a.NBLK = (ln[l] + CR - 1) / CR;
        a.total = (int64_t)s.B * a.NBLK * s.H_kv * 32;
        a.plane = (int64_t)s.B * a.NBLK * s.H_kv * CR * D;
        const unsigned grid = (unsigned)((a.total + 255) / 256);
        if (s.dtype == HTREE_F32) { if (CR == 16) block_values_kernel<64, 16, true><<<grid, 256, 0, st>>>(a); else block_values_kernel<64, 8, true><<<grid, 256, 0, st>>>(a); }
        else if (D == 128) { if (CR == 16) block_values_kernel<128, 16, false><<<grid, 256, 0, st>>>(a); else block_values_kernel<128, 8, false><<<grid, 256, 0, st>>>(a); }
        else { if (CR == 16) block_values_kernel<64, 16, false><<<grid, 256, 0, st>>>(a); else block_values_kernel<64, 8, false><<<grid, 256, 0, st>>>(a); }
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

struct TreeBwdArgs {
    const float* dparent[2];   // NULL: no parent level (the pass only casts)
    float* dchild[2];
    void* typed[2];            // NULL: the sum is written back to dchild; else it is written here in the storage type
    int32_t wv[2];     // float4 per row
    int64_t total[2];  // B * Nc * wv
    int32_t Nc, Np, CR;
};

// dchild[b, c, :] += dparent[b, c / CR, :] / count(c / CR): one float4 of a child row per thread.  With a typed
// destination (the last pass of a backward whose caller wants the gradients in the storage type) the sum goes there
// instead, rounded once: the cast of src/backward.py:1193 without another pass over the tensor.
template <typename TO>
__global__ void __launch_bounds__(256) tree_backward_kernel(const __grid_constant__ TreeBwdArgs a) {
    const int which = blockIdx.y;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total[which]) return;
    const int wv = a.wv[which];
    const int col = (int)(idx % wv);
    const int64_t row = idx / wv;   // b * Nc + c
    float4* dst = reinterpret_cast<float4*>(a.dchild[which]) + idx;
    float4 x = *dst;
    if (a.dparent[which]) {
        const int c = (int)(row % a.Nc);
        const int64_t b = row / a.Nc;
        const int p = c / a.CR;
        const float cnt = (float)min(a.CR, a.Nc - p * a.CR);
        const float4 g = __ldg(reinterpret_cast<const float4*>(a.dparent[which]) + ((b * a.Np + p) * (int64_t)wv + col));
        x.x += g.x / cnt; x.y += g.y / cnt; x.z += g.z / cnt; x.w += g.w / cnt;
    }
    if (a.typed[which]) {
        TO* o = reinterpret_cast<TO*>(a.typed[which]) + idx * 4;
        if (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(o) = x;
        } else {
            TO h[4] = {from_f<TO>(x.x), from_f<TO>(x.y), from_f<TO>(x.z), from_f<TO>(x.w)};
            *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(h);
        }
    } else {
        *dst = x;
    }
}

template <typename TO>
static int tree_backward_levels(const HtreeShape& s, int L, const int32_t* ln, float* const* dk, float* const* dv, cudaStream_t st,
                                void* typed_dk, void* typed_dv) {
    const bool typed = typed_dk != nullptr || typed_dv != nullptr;
    for (int l = L - 1; l >= (typed ? 0 : 1); --l) {
        // l >= 1: fold level l into level l-1; l == 0 (only with typed outputs and a single level): cast alone
        const int child = l >= 1 ? l - 1 : 0;
        TreeBwdArgs a;
        a.dparent[0] = l >= 1 ? dk[l] : nullptr; a.dparent[1] = l >= 1 ? dv[l] : nullptr;
        a.dchild[0] = dk[child]; a.dchild[1] = dv[child];
        const bool last = child == 0;
        a.typed[0] = last ? typed_dk : nullptr; a.typed[1] = last ? typed_dv : nullptr;
        a.wv[0] = s.H_kv * s.K / 4; a.wv[1] = s.H_kv * s.V / 4;
        a.Nc = ln[child]; a.Np = l >= 1 ? ln[l] : 1; a.CR = s.compression_rate;
        a.total[0] = (int64_t)s.B * a.Nc * a.wv[0]; a.total[1] = (int64_t)s.B * a.Nc * a.wv[1];
        int64_t mx = a.total[0] > a.total[1] ? a.total[0] : a.total[1];
        dim3 grid((unsigned)((mx + 255) / 256), 2);
        tree_backward_kernel<TO><<<grid, 256, 0, st>>>(a);
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
        if (l == 1 || l == 0) break;
    }
    return 0;
}

int launch_tree_backward(const HtreeShape& s, int L, const int32_t* ln, float* const* dk, float* const* dv, cudaStream_t st,
                         void* typed_dk, void* typed_dv) {
    switch (s.dtype) {
        case HTREE_BF16: return tree_backward_levels<__nv_bfloat16>(s, L, ln, dk, dv, st, typed_dk, typed_dv);
        case HTREE_F16: return tree_backward_levels<__half>(s, L, ln, dk, dv, st, typed_dk, typed_dv);
        default: return tree_backward_levels<float>(s, L, ln, dk, dv, st, typed_dk, typed_dv);
    }
}

}  // namespace htree
