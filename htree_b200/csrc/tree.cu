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
        if (s.compression_rate >= 16) tree_build_kernel<T, 16><<<grid, 256, 0, st>>>(a);
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

struct TreeBwdArgs {
    const float* dparent[2];
    float* dchild[2];
    int32_t wv[2];     // float4 per row
    int64_t total[2];  // B * Nc * wv
    int32_t Nc, Np, CR;
};

// dchild[b, c, :] += dparent[b, c / CR, :] / count(c / CR): one float4 of a child row per thread.
__global__ void __launch_bounds__(256) tree_backward_kernel(const __grid_constant__ TreeBwdArgs a) {
    const int which = blockIdx.y;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total[which]) return;
    const int wv = a.wv[which];
    const int col = (int)(idx % wv);
    const int64_t row = idx / wv;   // b * Nc + c
    const int c = (int)(row % a.Nc);
    const int64_t b = row / a.Nc;
    const int p = c / a.CR;
    const float cnt = (float)min(a.CR, a.Nc - p * a.CR);
    const float4 g = __ldg(reinterpret_cast<const float4*>(a.dparent[which]) + ((b * a.Np + p) * (int64_t)wv + col));
    float4* dst = reinterpret_cast<float4*>(a.dchild[which]) + idx;
    float4 x = *dst;
    x.x += g.x / cnt; x.y += g.y / cnt; x.z += g.z / cnt; x.w += g.w / cnt;
    *dst = x;
}

int launch_tree_backward(const HtreeShape& s, int L, const int32_t* ln, float* const* dk, float* const* dv, cudaStream_t st) {
    for (int l = L - 1; l >= 1; --l) {
        TreeBwdArgs a;
        a.dparent[0] = dk[l]; a.dparent[1] = dv[l];
        a.dchild[0] = dk[l - 1]; a.dchild[1] = dv[l - 1];
        a.wv[0] = s.H_kv * s.K / 4; a.wv[1] = s.H_kv * s.V / 4;
        a.Nc = ln[l - 1]; a.Np = ln[l]; a.CR = s.compression_rate;
        a.total[0] = (int64_t)s.B * a.Nc * a.wv[0]; a.total[1] = (int64_t)s.B * a.Nc * a.wv[1];
        int64_t mx = a.total[0] > a.total[1] ? a.total[0] : a.total[1];
        dim3 grid((unsigned)((mx + 255) / 256), 2);
        tree_backward_kernel<<<grid, 256, 0, st>>>(a);
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

}  // namespace htree
