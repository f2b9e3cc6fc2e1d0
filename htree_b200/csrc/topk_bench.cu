// Stand-alone Top-K selectors for the selector micro-benchmark (the experiment of topk_test/benchmark.py:34-46 of the
// reference: `batch` independent problems, the k largest of n fp32 values each, with 0, 1 or 8 int32 payload words
// carried along).  One thread block per problem, all keys in shared memory.  Three selectors:
//   0  threshold search   the selector of the attention kernels (fwd_generic.cu / fwd_mma.cu): a 32-step bitwise search
//                         for the k-th largest key by counting, then a scan that emits the winners in index order
//   1  radix select       four 8-bit digit histograms narrow the k-th largest key, then the same emit step
//   2  bitonic            sort k-element runs, then halve: pairwise maxima of a descending and an ascending run are the
//                         top k of both and form a bitonic run again; output sorted by value
// Ties go to the smaller index in all three.  Selectors 0 and 1 return indices ascending (what the attention kernels
// need: the kept nodes are the next level's parent list); selector 2 returns them by descending value.
#include "common.cuh"

namespace htree {

constexpr int TKN = 512;            // threads per block
constexpr int TK_MAX_N = 8192;      // keys held in shared memory

__device__ __forceinline__ uint32_t ordered_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return u ^ ((u >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

__device__ __forceinline__ int block_sum(int v, int* red) {
    v = __reduce_add_sync(0xffffffffu, v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    int s = 0;
#pragma unroll
    for (int w = 0; w < TKN / 32; ++w) s += red[w];
    return s;
}

struct TopkArgs {
    const float* values; const int32_t* pay1; const int32_t* pay8;
    float* out_val; int32_t* out_idx; int32_t* out_pay1; int32_t* out_pay8;
    int n, k;
};

__device__ __forceinline__ void write_winner(const TopkArgs& a, int64_t prob, int slot, int idx, float val) {
    const int64_t o = prob * a.k + slot;
    a.out_val[o] = val;
    a.out_idx[o] = idx;
    if (a.pay1) a.out_pay1[o] = a.pay1[prob * a.n + idx];
    if (a.pay8) {
        const int4* src = reinterpret_cast<const int4*>(a.pay8 + (prob * a.n + idx) * 8);
        int4* dst = reinterpret_cast<int4*>(a.out_pay8 + o * 8);
        dst[0] = src[0];
        dst[1] = src[1];
    }
}

// Winners = keys above thr plus the first `need` keys equal to thr, emitted in ascending index order: every warp owns a
// contiguous segment, counts its winners, and ranks them with ballots on a second walk.
__device__ void emit_in_index_order(const TopkArgs& a, int64_t prob, const uint32_t* key, uint32_t thr, int need, int* red) {
    constexpr int NW = TKN / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = (a.n + NW - 1) / NW, lo = warp * seg, hi = min(a.n, lo + seg);
    int gt = 0, eq = 0;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const uint32_t kj = j < hi ? key[j] : 0u;
        gt += __popc(__ballot_sync(0xffffffffu, j < hi && kj > thr));
        eq += __popc(__ballot_sync(0xffffffffu, j < hi && kj == thr));
    }
    __syncthreads();
    if (lane == 0) red[warp] = gt | (eq << 16);
    __syncthreads();
    int gt_b = 0, eq_b = 0;
    for (int w = 0; w < warp; ++w) { gt_b += red[w] & 0xFFFF; eq_b += red[w] >> 16; }
    const uint32_t below = (1u << lane) - 1u;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const uint32_t kj = j < hi ? key[j] : 0u;
        const bool is_gt = j < hi && kj > thr, is_eq = j < hi && kj == thr;
        const uint32_t bg = __ballot_sync(0xffffffffu, is_gt), be = __ballot_sync(0xffffffffu, is_eq);
        const int g_rank = gt_b + __popc(bg & below), e_rank = eq_b + __popc(be & below);
        if (is_gt) write_winner(a, prob, g_rank + min(e_rank, need), j, key_value(kj));
        else if (is_eq && e_rank < need) write_winner(a, prob, g_rank + e_rank, j, key_value(kj));
        gt_b += __popc(bg);
        eq_b += __popc(be);
    }
}

__global__ void __launch_bounds__(TKN) topk_threshold_kernel(const TopkArgs a) {
    extern __shared__ uint32_t key[];
    __shared__ int red[TKN / 32];
    const int64_t prob = blockIdx.x;
    for (int j = threadIdx.x; j < a.n; j += TKN) key[j] = ordered_key(a.values[prob * a.n + j]);
    __syncthreads();
    uint32_t thr = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const uint32_t cand = thr | (1u << bit);
        int c = 0;
        for (int j = threadIdx.x; j < a.n; j += TKN) c += key[j] >= cand;
        const int n_ge = block_sum(c, red);
        if (n_ge >= a.k) thr = cand;
        if (n_ge == a.k) break;   // the winner set is decided: lower bits cannot change it
    }
    int c = 0;
    for (int j = threadIdx.x; j < a.n; j += TKN) c += key[j] > thr;
    const int need = a.k - block_sum(c, red);
    emit_in_index_order(a, prob, key, thr, need, red);
}

__global__ void __launch_bounds__(TKN) topk_radix_kernel(const TopkArgs a) {
    extern __shared__ uint32_t key[];
    __shared__ int red[TKN / 32];
    __shared__ int hist[256];
    __shared__ int pick[2];       // chosen digit, winners still to find among the keys that share the prefix
    const int64_t prob = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int j = tid; j < a.n; j += TKN) key[j] = ordered_key(a.values[prob * a.n + j]);
    uint32_t prefix = 0, fixed = 0;   // digits decided so far and their mask
    int want = a.k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int j = tid; j < a.n; j += TKN) {
            const uint32_t kj = key[j];
            if (((kj ^ prefix) & fixed) == 0) atomicAdd(&hist[(kj >> shift) & 255u], 1);
        }
        __syncthreads();
        // suffix sums over the digits, largest digit first: thread i looks at digit 255 - i
        int v = 0, inc = 0;
        if (tid < 256) {
            v = hist[255 - tid];
            inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += y;
            }
            if (lane == 31) red[warp] = inc;
        }
        __syncthreads();
        if (tid < 256) {
            for (int w = 0; w < warp; ++w) inc += red[w];
            const int exc = inc - v;
            if (exc < want && want <= inc) { pick[0] = 255 - tid; pick[1] = want - exc; }
        }
        __syncthreads();
        prefix |= (uint32_t)pick[0] << shift;
        fixed |= 255u << shift;
        want = pick[1];
        __syncthreads();
    }
    emit_in_index_order(a, prob, key, prefix, want, red);
}

// (key, ~index) as one 64-bit word: descending order of the word = descending value, ties to the smaller index.
__device__ __forceinline__ void compare_exchange(uint64_t* x, int i, int j, bool descending) {
    const uint64_t u = x[i], w = x[j];
    if ((u < w) == descending) { x[i] = w; x[j] = u; }
}

__global__ void __launch_bounds__(TKN) topk_bitonic_kernel(const TopkArgs a) {
    extern __shared__ uint64_t x[];
    const int64_t prob = blockIdx.x;
    const int n = a.n, k = a.k, tid = threadIdx.x;
    for (int j = tid; j < n; j += TKN)
        x[j] = ((uint64_t)ordered_key(a.values[prob * n + j]) << 32) | (uint32_t)~(uint32_t)j;
    __syncthreads();
    // runs of k, even runs descending, odd runs ascending
    for (int size = 2; size <= k; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n / 2; i += TKN) {
                const int pos = 2 * i - (i & (stride - 1));
                compare_exchange(x, pos, pos + stride, (pos & size) == 0);
            }
            __syncthreads();
        }
    // halve: the maxima of a descending run and the ascending run after it are the top k of both (a bitonic run);
    // pack them to the front, then merge every run back into alternating order
    for (int m = n; m > k; m >>= 1) {
        constexpr int PER = TK_MAX_N / 2 / TKN;
        uint64_t keep[PER];
#pragma unroll
        for (int u_ = 0; u_ < PER; ++u_) {
            const int i = tid + u_ * TKN;
            if (i < m / 2) {
                const int run = i / k, off = i - run * k;
                const uint64_t u = x[2 * run * k + off], w = x[(2 * run + 1) * k + off];
                keep[u_] = u > w ? u : w;
            }
        }
        __syncthreads();
#pragma unroll
        for (int u_ = 0; u_ < PER; ++u_) {
            const int i = tid + u_ * TKN;
            if (i < m / 2) x[i] = keep[u_];
        }
        __syncthreads();
        for (int stride = k >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < m / 4; i += TKN) {
                const int pos = 2 * i - (i & (stride - 1));
                compare_exchange(x, pos, pos + stride, (pos & k) == 0);
            }
            __syncthreads();
        }
    }
    for (int j = tid; j < k; j += TKN) {
        const uint64_t u = x[j];
        write_winner(a, prob, j, (int)~(uint32_t)u, key_value((uint32_t)(u >> 32)));
    }
}

int launch_topk(const TopkArgs& a, int batch, int method, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    if (method == 0) {
        topk_threshold_kernel<<<batch, TKN, a.n * sizeof(uint32_t), st>>>(a);
    } else if (method == 1) {
        topk_radix_kernel<<<batch, TKN, a.n * sizeof(uint32_t), st>>>(a);
    } else {
        const size_t smem = a.n * sizeof(uint64_t);
        e = cudaFuncSetAttribute(topk_bitonic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        topk_bitonic_kernel<<<batch, TKN, smem, st>>>(a);
    }
    note_launch();
    return (int)cudaGetLastError();
}

}  // namespace htree

extern "C" int htree_b200_topk(const float* values, const int32_t* pay1, const int32_t* pay8, int32_t batch, int32_t n,
                               int32_t k, int32_t method, float* out_val, int32_t* out_idx, int32_t* out_pay1,
                               int32_t* out_pay8, void* stream) {
    using namespace htree;
    if (!values || !out_val || !out_idx) return HTREE_E_NULL;
    if ((pay1 && !out_pay1) || (pay8 && !out_pay8)) return HTREE_E_NULL;
    if (batch <= 0 || n <= 0 || k <= 0 || k > n) return HTREE_E_SHAPE;
    if (n > TK_MAX_N || method < 0 || method > 2) return HTREE_E_UNSUPPORTED;
    if (method == 2 && ((n & (n - 1)) || (k & (k - 1)) || k < 2)) return HTREE_E_UNSUPPORTED;   // the network needs powers of two
    if (pay8 && (((uintptr_t)pay8 | (uintptr_t)out_pay8) & 15u)) return HTREE_E_ALIGN;   // payload rows move as 16-byte words
    TopkArgs a{values, pay1, pay8, out_val, out_idx, out_pay1, out_pay8, n, k};
    return launch_topk(a, batch, method, (cudaStream_t)stream);
}
