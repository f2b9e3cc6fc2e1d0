// Shared declarations of the htree_b200 kernels: parameter blocks, storage-type helpers, block primitives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/htree_b200.h"

namespace htree {

constexpr float kNegInf = -1.0e10f;      // HTREE_SCORE_NEG_INF of the reference (src/parallel.py:75)
constexpr float kHasMass = 1.0e-10f;     // "has contribution" guard of the level merge (src/parallel.py:289-314)
constexpr float kForcedImportance = 1.0e6f;  // importance given to the right-most candidate (src/parallel.py:745)

// Everything the attention kernels need, passed by value as a __grid_constant__ block.
struct AttnParams {
    const void* q;
    const void* lk[HTREE_MAX_LEVELS];
    const void* lv[HTREE_MAX_LEVELS];
    const void* lkr[HTREE_MAX_LEVELS];   // keys pre-rotated by their child index (16-bit storage types only), or NULL
    const void* lvb[HTREE_MAX_LEVELS];   // values re-laid-out per parent block for the P.V fragments (tree.cu), or NULL
    const void* lkb[HTREE_MAX_LEVELS];   // pre-rotated keys per parent block in fragment-major order (tree.cu), or NULL
    int32_t ln[HTREE_MAX_LEVELS];   // N_l
    int64_t lpow[HTREE_MAX_LEVELS]; // CR^l
    const float* cosc;
    const float* sinc;
    const __half* cosh;   // optional: cos * scale and sin * scale as IEEE half, same shape as cosc/sinc
    const __half* sinh;
    int32_t* parents[HTREE_MAX_LEVELS];  // may be all NULL in the forward
    int32_t* status;
    // forward outputs
    void* out;
    float* gmax;
    float* gsum;
    float* tr_max;
    float* tr_sum;
    float* tr_out;
    // backward inputs / outputs
    const void* dO;
    float* dq;          // fp32 dq (the reference's contract), or NULL when dq_typed is set
    void* dq_typed;     // dq in the storage type of q, or NULL
    float* dk[HTREE_MAX_LEVELS];
    float* dv[HTREE_MAX_LEVELS];
    int32_t B, T, H, Hkv, K, V, CR, TK, L, G, n_pos;
    // single-level mode of the generic forward (per-kernel compatibility surface): only level `level_index` runs, its
    // parent lists come from parents_in and the kept nodes go to next_out; the per-level state goes to tr_* slot 0
    const int32_t* parents_in;
    int32_t* next_out;
    int32_t level_mode, level_index;
    int32_t Tq, t0;   // query window: rows 0..Tq-1 of q/out are sequence positions t0..t0+Tq-1
    float scale;
    uint32_t flags;
};

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// Four consecutive elements as floats with one vector load (pointer must be aligned to 4 elements).
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&o)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&o)[4]) {
    float4 x = __ldg(reinterpret_cast<const float4*>(p));
    o[0] = x.x; o[1] = x.y; o[2] = x.z; o[3] = x.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[4]) {
    uint2 x = __ldg(reinterpret_cast<const uint2*>(p));
    o[0] = __uint_as_float(x.x << 16); o[1] = __uint_as_float(x.x & 0xffff0000u);
    o[2] = __uint_as_float(x.y << 16); o[3] = __uint_as_float(x.y & 0xffff0000u);
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&o)[4]) {
    uint2 x = __ldg(reinterpret_cast<const uint2*>(p));
    float2 a = __half22float2(*reinterpret_cast<__half2*>(&x.x));
    float2 b = __half22float2(*reinterpret_cast<__half2*>(&x.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Exclusive scan of one flag per thread over the block, in thread order.  `wtot` is shared scratch of NT/32 ints.
// Returns the number of set flags in lower threads; *total receives the block total.  Two barriers.
template <int NT>
__device__ __forceinline__ int block_scan_flag(bool f, int* wtot, int* total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    unsigned m = __ballot_sync(0xffffffffu, f);
    if (lane == 0) wtot[w] = __popc(m);
    __syncthreads();
    int before = 0, tot = 0;
#pragma unroll
    for (int i = 0; i < NT / 32; ++i) {
        int c = wtot[i];
        if (i < w) before += c;
        tot += c;
    }
    __syncthreads();
    *total = tot;
    return before + __popc(m & ((1u << lane) - 1u));
}

void note_launch(int n = 1);   // diagnostic launch counter (api.cu)

// Parent lists: int32 with -1 for "none" (the reference's layout), or uint16 with 0xFFFF under HTREE_PARENTS_U16.
__device__ __forceinline__ int load_parent(const AttnParams& p, int l, int64_t idx) {
    if (p.flags & HTREE_PARENTS_U16) {
        const uint16_t v = reinterpret_cast<const uint16_t*>(p.parents[l])[idx];
        return v == 0xFFFFu ? -1 : (int)v;
    }
    return p.parents[l][idx];
}
__device__ __forceinline__ void store_parent(const AttnParams& p, int l, int64_t idx, int v) {
    if (p.flags & HTREE_PARENTS_U16) reinterpret_cast<uint16_t*>(p.parents[l])[idx] = v < 0 ? (uint16_t)0xFFFFu : (uint16_t)v;
    else p.parents[l][idx] = v;
}

// launchers implemented in the .cu files (return cudaError_t as int)
int launch_tree_build(const HtreeShape& s, int L, const int32_t* ln, void* const* lk, void* const* lv, cudaStream_t st);
// typed_dk / typed_dv: NULL, or buffers of the storage type that receive the finished leaf gradients (the cast is fused
// into the last streaming pass; the fp32 level-0 buffers then only hold the accumulators)
int launch_tree_backward(const HtreeShape& s, int L, const int32_t* ln, float* const* dk, float* const* dv, cudaStream_t st,
                         void* typed_dk = nullptr, void* typed_dv = nullptr);
int launch_rotate_keys(const HtreeShape& s, int L, const int32_t* ln, void* const* lk, void* const* lkr, const float* cosc,
                       const float* sinc, cudaStream_t st);
int launch_fwd_generic(const AttnParams& p, int dtype, cudaStream_t st);
int launch_merge_to_global(const float* lmax, const float* lsum, const float* lout, float* gmax, float* gsum, float* gout,
                           int64_t rows, int V, cudaStream_t st);
int launch_final_normalize(const float* gout, const float* gsum, void* out, int dtype, int64_t rows, int V, cudaStream_t st);
int launch_block_values(const HtreeShape& s, int L, const int32_t* ln, void* const* lv, void* const* lvb, cudaStream_t st);
int launch_block_keys(const HtreeShape& s, int L, const int32_t* ln, void* const* lkr, void* const* lkb, cudaStream_t st);

// Element order inside a block of the blocked values: fragment-major ([16-byte piece][lane]) for 128-wide heads with 16
// children per parent and a 16-bit storage type (read through shared memory by the pipelined forward), lane-major
// (each lane's pieces consecutive) otherwise.
template <int D, int CR, bool SPLIT>
constexpr bool kFragmentMajor = (D == 128 && CR == 16 && !SPLIT);
bool fwd_mma_supported(const AttnParams& p, int dtype);
int launch_fwd_mma(const AttnParams& p, int dtype, cudaStream_t st);
bool bwd_mma_supported(const AttnParams& p, int dtype);
int launch_bwd_mma(const AttnParams& p, int dtype, cudaStream_t st);
bool bwd_generic_supported(const AttnParams& p, int dtype);
int launch_bwd_generic(const AttnParams& p, int dtype, cudaStream_t st);

}  // namespace htree
