// extern "C" boundary of libhtree_b200: argument validation, parameter blocks, kernel dispatch.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace htree {

static std::atomic<unsigned long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

static int esize(int dtype) { return dtype == HTREE_F32 ? 4 : 2; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// the tensor-core kernels move 32-byte pieces with 256-bit loads
static bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

static int level_sizes(int T, int CR, int MTN, int32_t* ln) {
    if (T <= 0 || CR < 2 || MTN < 1) return HTREE_E_SHAPE;
    int L = 1, n = T;
    ln[0] = T;
    while (n > MTN) {
        n = (n + CR - 1) / CR;
        if (L >= HTREE_MAX_LEVELS) return HTREE_E_LEVELS;
        ln[L++] = n;
    }
    return L;
}

static int check_shape(const HtreeShape* s, int32_t* ln, bool check_top = true) {
    if (!s) return HTREE_E_NULL;
    if (s->B <= 0 || s->T <= 0 || s->H <= 0 || s->H_kv <= 0 || s->K <= 0 || s->V <= 0 || s->top_k <= 0) return HTREE_E_SHAPE;
    if (s->H % s->H_kv != 0 || (s->K & 1)) return HTREE_E_SHAPE;
    if (s->dtype != HTREE_F32 && s->dtype != HTREE_BF16 && s->dtype != HTREE_F16) return HTREE_E_DTYPE;
    if ((int64_t)s->B * s->H_kv > 65535) return HTREE_E_UNSUPPORTED;
    const int L = level_sizes(s->T, s->compression_rate, s->max_top_nodes, ln);
    if (L < 0) return L;
    if (check_top && (int64_t)ln[L - 1] > (int64_t)s->top_k * s->compression_rate) return HTREE_E_TOPLEVEL;
    // 16-byte rows: K, V multiples of 8 keep every vector load of every kernel aligned for all storage types
    if (s->K % 8 != 0 || s->V % 8 != 0) return HTREE_E_ALIGN;
    if (s->T_q < 0 || s->t_offset < 0 || (s->T_q == 0 && s->t_offset != 0) ||
        (int64_t)s->t_offset + s->T_q > s->T) return HTREE_E_WINDOW;
    return L;
}

static int fill_params(AttnParams& p, const HtreeShape* s, int L, const int32_t* ln, const void* q, void* const* lk,
                       void* const* lv, const float* cosc, const float* sinc, int32_t n_pos, float scale,
                       int32_t* const* parents, int32_t* status, uint32_t flags) {
    std::memset(&p, 0, sizeof(p));
    if (!q || !lk || !lv || !cosc || !sinc) return HTREE_E_NULL;
    if ((int64_t)n_pos < (int64_t)s->top_k * s->compression_rate) return HTREE_E_ROPE;
    if (!aligned16(q) || !aligned16(cosc) || !aligned16(sinc)) return HTREE_E_ALIGN;
    if ((flags & HTREE_PARENTS_U16) && parents) {   // ids of level l+1 (or of the virtual parents) must fit, 0xFFFF = none
        if (s->top_k > 65535) return HTREE_E_UNSUPPORTED;
        for (int l = 1; l < L; ++l) if (ln[l] > 65535) return HTREE_E_UNSUPPORTED;
    }
    p.q = q;
    int64_t pw = 1;
    for (int l = 0; l < L; ++l) {
        if (!lk[l] || !lv[l]) return HTREE_E_NULL;
        if (!aligned16(lk[l]) || !aligned16(lv[l])) return HTREE_E_ALIGN;
        p.lk[l] = lk[l]; p.lv[l] = lv[l]; p.ln[l] = ln[l]; p.lpow[l] = pw;
        p.parents[l] = parents ? parents[l] : nullptr;
        pw *= s->compression_rate;
    }
    p.cosc = cosc; p.sinc = sinc; p.status = status;
    p.B = s->B; p.T = s->T; p.H = s->H; p.Hkv = s->H_kv; p.K = s->K; p.V = s->V;
    p.CR = s->compression_rate; p.TK = s->top_k; p.L = L; p.G = s->H / s->H_kv; p.n_pos = n_pos;
    p.Tq = s->T_q > 0 ? s->T_q : s->T; p.t0 = s->t_offset;
    p.scale = scale; p.flags = flags;
    return 0;
}

}  // namespace htree

using namespace htree;

extern "C" {

int htree_b200_version(void) { return HTREE_B200_VERSION; }

uint64_t htree_b200_launch_count(void) { return (uint64_t)htree::g_launches.load(std::memory_order_relaxed); }

const char* htree_b200_error_string(int code) {
    switch (code) {
        case 0: return "success";
        case HTREE_E_NULL: return "a required pointer is NULL";
        case HTREE_E_SHAPE: return "invalid shape: sizes must be positive, H divisible by H_kv, K even";
        case HTREE_E_DTYPE: return "unknown storage type";
        case HTREE_E_LEVELS: return "too many tree levels";
        case HTREE_E_TOPLEVEL: return "top tree level is longer than top_k*compression_rate";
        case HTREE_E_ROPE: return "cos/sin tables have fewer than top_k*compression_rate rows";
        case HTREE_E_ALIGN: return "pointers must be 16-byte aligned and K, V multiples of 8";
        case HTREE_E_UNSUPPORTED: return "shape not supported by the compiled kernels";
        case HTREE_E_NODEVICE: return "no usable CUDA device";
        case HTREE_E_WINDOW: return "query window outside the sequence, or a backward window without HTREE_BWD_KEEP_ACCUM / HTREE_BWD_NO_FOLD";
        case HTREE_E_SCRATCH: return "pooled tree levels do not fit the built-in scratch array (see htree_b200_static_scratch_bytes)";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown htree_b200 error";
    }
}

int htree_b200_num_levels(int32_t T, int32_t CR, int32_t MTN) {
    int32_t ln[HTREE_MAX_LEVELS];
    return level_sizes(T, CR, MTN, ln);
}

int htree_b200_level_sizes(int32_t T, int32_t CR, int32_t MTN, int32_t* sizes, int32_t cap) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = level_sizes(T, CR, MTN, ln);
    if (L < 0) return L;
    if (!sizes) return HTREE_E_NULL;
    for (int l = 0; l < L && l < cap; ++l) sizes[l] = ln[l];
    return L;
}

int htree_b200_build_tree(const HtreeShape* shape, void* const* layers_k, void* const* layers_v,
                          void* const* layers_k_rot, void* const* layers_k_blk, void* const* layers_v_blk,
                          const float* cos_cache, const float* sin_cache, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln, false);   // top_k plays no role in the tree
    if (L < 0) return L;
    if (!layers_k || !layers_v) return HTREE_E_NULL;
    for (int l = 0; l < L; ++l) {
        if (!layers_k[l] || !layers_v[l]) return HTREE_E_NULL;
        if (!aligned16(layers_k[l]) || !aligned16(layers_v[l])) return HTREE_E_ALIGN;
    }
    const int es = esize(shape->dtype);
    if ((shape->H_kv * shape->K * es) % 16 || (shape->H_kv * shape->V * es) % 16) return HTREE_E_ALIGN;
    if (layers_k_rot) {
        if (!cos_cache || !sin_cache) return HTREE_E_NULL;
        if (!aligned16(cos_cache) || !aligned16(sin_cache)) return HTREE_E_ALIGN;
        for (int l = 0; l < L; ++l) {
            if (!layers_k_rot[l]) return HTREE_E_NULL;
            if (!aligned16(layers_k_rot[l])) return HTREE_E_ALIGN;
        }
    }
    if (layers_v_blk) {
        if ((shape->V != 64 && shape->V != 128) || (shape->compression_rate != 8 && shape->compression_rate != 16) ||
            (shape->dtype == HTREE_F32 && shape->V != 64))
            return HTREE_E_UNSUPPORTED;
        for (int l = 0; l < L; ++l) {
            if (!layers_v_blk[l]) return HTREE_E_NULL;
            if (!aligned32(layers_v_blk[l])) return HTREE_E_ALIGN;
        }
    }
    if (layers_k_blk) {
        if (!layers_k_rot) return HTREE_E_NULL;       // the blocked keys are built from the rotated keys
        if (shape->dtype == HTREE_F32 || shape->K != 128 || shape->compression_rate != 16) return HTREE_E_UNSUPPORTED;
        for (int l = 0; l < L; ++l) {
            if (!layers_k_blk[l]) return HTREE_E_NULL;
            if (!aligned32(layers_k_blk[l])) return HTREE_E_ALIGN;
        }
    }
    int rc = launch_tree_build(*shape, L, ln, layers_k, layers_v, (cudaStream_t)stream);
    if (rc == 0 && layers_k_rot)
        rc = launch_rotate_keys(*shape, L, ln, layers_k, layers_k_rot, cos_cache, sin_cache, (cudaStream_t)stream);
    if (rc == 0 && layers_k_blk)
        rc = launch_block_keys(*shape, L, ln, layers_k_rot, layers_k_blk, (cudaStream_t)stream);
    if (rc == 0 && layers_v_blk)
        rc = launch_block_values(*shape, L, ln, layers_v, layers_v_blk, (cudaStream_t)stream);
    return rc;
}

int htree_b200_block_keys(const HtreeShape* shape, void* const* layers_k_rot, void* const* layers_k_blk, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln, false);
    if (L < 0) return L;
    if (!layers_k_rot || !layers_k_blk) return HTREE_E_NULL;
    if (shape->dtype == HTREE_F32 || shape->K != 128 || shape->compression_rate != 16) return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L; ++l) {
        if (!layers_k_rot[l] || !layers_k_blk[l]) return HTREE_E_NULL;
        if (!aligned16(layers_k_rot[l]) || !aligned32(layers_k_blk[l])) return HTREE_E_ALIGN;
    }
    return launch_block_keys(*shape, L, ln, layers_k_rot, layers_k_blk, (cudaStream_t)stream);
}

int htree_b200_block_values(const HtreeShape* shape, void* const* layers_v, void* const* layers_v_blk, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln, false);
    if (L < 0) return L;
    if (!layers_v || !layers_v_blk) return HTREE_E_NULL;
    if ((shape->V != 64 && shape->V != 128) || (shape->compression_rate != 8 && shape->compression_rate != 16) ||
        (shape->dtype == HTREE_F32 && shape->V != 64))
        return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L; ++l) {
        if (!layers_v[l] || !layers_v_blk[l]) return HTREE_E_NULL;
        if (!aligned16(layers_v[l]) || !aligned32(layers_v_blk[l])) return HTREE_E_ALIGN;
    }
    return launch_block_values(*shape, L, ln, layers_v, layers_v_blk, (cudaStream_t)stream);
}

int htree_b200_rotate_keys(const HtreeShape* shape, void* const* layers_k, void* const* layers_k_rot,
                           const float* cos_cache, const float* sin_cache, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln, false);
    if (L < 0) return L;
    if (!layers_k || !layers_k_rot || !cos_cache || !sin_cache) return HTREE_E_NULL;
    if (!aligned16(cos_cache) || !aligned16(sin_cache)) return HTREE_E_ALIGN;
    for (int l = 0; l < L; ++l) {
        if (!layers_k[l] || !layers_k_rot[l]) return HTREE_E_NULL;
        if (!aligned16(layers_k[l]) || !aligned16(layers_k_rot[l])) return HTREE_E_ALIGN;
    }
    return launch_rotate_keys(*shape, L, ln, layers_k, layers_k_rot, cos_cache, sin_cache, (cudaStream_t)stream);
}

int htree_b200_forward(const HtreeShape* shape, const void* q, void* const* layers_k, void* const* layers_v,
                       void* const* layers_k_rot, void* const* layers_k_blk, void* const* layers_v_blk, const float* cos_cache,
                       const float* sin_cache, const void* cos_half,
                       const void* sin_half, int32_t n_pos, float scale, void* out,
                       float* gmax, float* gsum, int32_t* const* parents, const HtreeTrace* trace, int32_t* status,
                       uint32_t flags, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln);
    if (L < 0) return L;
    AttnParams p;
    int rc = fill_params(p, shape, L, ln, q, layers_k, layers_v, cos_cache, sin_cache, n_pos, scale, parents, status, flags);
    if (rc) return rc;
    const bool select_only = (flags & HTREE_FWD_SELECT_ONLY) != 0;
    if (select_only) {
        if (!parents) return HTREE_E_NULL;
    } else {
        if (!out || !gmax || !gsum) return HTREE_E_NULL;
        if (!aligned16(out)) return HTREE_E_ALIGN;
    }
    p.out = out; p.gmax = gmax; p.gsum = gsum;
    if (cos_half && sin_half && aligned32(cos_half) && aligned32(sin_half)) {
        p.cosh = static_cast<const __half*>(cos_half); p.sinh = static_cast<const __half*>(sin_half);
    }
    if (trace) { p.tr_max = trace->layer_max; p.tr_sum = trace->layer_sum; p.tr_out = trace->layer_out; }
    if (layers_k_rot && !trace && !(flags & HTREE_FWD_GENERIC)) {
        bool all = true;
        for (int l = 0; l < L; ++l) {
            if (!layers_k_rot[l] || !aligned32(layers_k_rot[l])) all = false;
            p.lkr[l] = layers_k_rot[l];
            if (!select_only) {   // the accumulating passes read the blocked values
                if (!layers_v_blk || !layers_v_blk[l] || !aligned32(layers_v_blk[l])) all = false;
                else p.lvb[l] = layers_v_blk[l];
            }
            // optional: with the blocked keys of every level the pipelined kernels run (bulk copies need 16-byte alignment)
            if (layers_k_blk && layers_k_blk[l] && aligned32(layers_k_blk[l])) p.lkb[l] = layers_k_blk[l];
        }
        all = all && aligned32(q) && aligned32(cos_cache) && aligned32(sin_cache);
        if (all && fwd_mma_supported(p, shape->dtype)) return launch_fwd_mma(p, shape->dtype, (cudaStream_t)stream);
    }
    return launch_fwd_generic(p, shape->dtype, (cudaStream_t)stream);
}

int htree_b200_level_forward(const HtreeShape* s, int32_t level, int32_t n_level, const void* q, const void* layer_k,
                             const void* layer_v, const int32_t* prev_parents, const float* cos_cache,
                             const float* sin_cache, int32_t n_pos, float scale, float* layer_max, float* layer_sum,
                             float* layer_out, int32_t* next_parents, int32_t* status, void* stream) {
    if (!s || !q || !layer_k || !layer_v || !prev_parents || !cos_cache || !sin_cache || !layer_max || !layer_sum || !layer_out)
        return HTREE_E_NULL;
    if (s->B <= 0 || s->T <= 0 || s->H <= 0 || s->H_kv <= 0 || s->K <= 0 || s->V <= 0 || s->top_k <= 0 || n_level <= 0 ||
        s->compression_rate < 2 || s->H % s->H_kv != 0 || (s->K & 1))
        return HTREE_E_SHAPE;
    if (level < 0 || level >= HTREE_MAX_LEVELS) return HTREE_E_LEVELS;
    if (level > 0 && !next_parents) return HTREE_E_NULL;
    if (s->dtype != HTREE_F32 && s->dtype != HTREE_BF16 && s->dtype != HTREE_F16) return HTREE_E_DTYPE;
    if (s->K % 8 != 0 || s->V % 8 != 0 || !aligned16(q) || !aligned16(layer_k) || !aligned16(layer_v) || !aligned16(cos_cache) ||
        !aligned16(sin_cache))
        return HTREE_E_ALIGN;
    if ((int64_t)n_pos < (int64_t)s->top_k * s->compression_rate) return HTREE_E_ROPE;
    if ((int64_t)s->B * s->H_kv > 65535) return HTREE_E_UNSUPPORTED;
    AttnParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = q; p.lk[level] = layer_k; p.lv[level] = layer_v; p.ln[level] = n_level;
    int64_t pw = 1;
    for (int l = 0; l < level; ++l) pw *= s->compression_rate;
    p.lpow[level] = pw;
    p.cosc = cos_cache; p.sinc = sin_cache; p.status = status;
    p.B = s->B; p.T = s->T; p.H = s->H; p.Hkv = s->H_kv; p.K = s->K; p.V = s->V;
    p.CR = s->compression_rate; p.TK = s->top_k; p.L = level + 1; p.G = s->H / s->H_kv; p.n_pos = n_pos;
    p.Tq = s->T; p.t0 = 0; p.scale = scale; p.flags = 0;
    p.level_mode = 1; p.level_index = level; p.parents_in = prev_parents; p.next_out = next_parents;
    p.tr_max = layer_max; p.tr_sum = layer_sum; p.tr_out = layer_out;
    return launch_fwd_generic(p, s->dtype, (cudaStream_t)stream);
}

int htree_b200_merge_to_global(const float* layer_max, const float* layer_sum, const float* layer_out, float* global_max,
                               float* global_sum, float* global_out, int64_t rows, int32_t V, void* stream) {
    if (!layer_max || !layer_sum || !layer_out || !global_max || !global_sum || !global_out) return HTREE_E_NULL;
    if (rows <= 0 || V <= 0) return HTREE_E_SHAPE;
    return launch_merge_to_global(layer_max, layer_sum, layer_out, global_max, global_sum, global_out, rows, V, (cudaStream_t)stream);
}

int htree_b200_final_normalize(const float* global_out, const float* global_sum, void* out, int32_t dtype, int64_t rows,
                               int32_t V, void* stream) {
    if (!global_out || !global_sum || !out) return HTREE_E_NULL;
    if (rows <= 0 || V <= 0) return HTREE_E_SHAPE;
    if (dtype != HTREE_F32 && dtype != HTREE_BF16 && dtype != HTREE_F16) return HTREE_E_DTYPE;
    return launch_final_normalize(global_out, global_sum, out, dtype, rows, V, (cudaStream_t)stream);
}

int htree_b200_copy_rows(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                         void* stream) {
    if (!dst || !src) return HTREE_E_NULL;
    if (width <= 0 || height <= 0 || dpitch < width || spitch < width) return HTREE_E_SHAPE;
    return (int)cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width, (size_t)height, cudaMemcpyDefault,
                                  (cudaStream_t)stream);
}

int htree_b200_backward(const HtreeShape* shape, const void* q, void* const* layers_k, void* const* layers_v,
                        void* const* layers_k_rot, const float* cos_cache, const float* sin_cache, const void* cos_half,
                        const void* sin_half, int32_t n_pos, float scale, const void* out,
                        const void* dO, const float* gmax, const float* gsum, int32_t* const* parents, float* dq,
                        float* const* dk_levels, float* const* dv_levels, const HtreeTypedGrads* typed, int32_t* status,
                        uint32_t flags, void* stream) {
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = check_shape(shape, ln);
    if (L < 0) return L;
    if (!out || !dO || !gmax || !gsum || !parents || !dk_levels || !dv_levels) return HTREE_E_NULL;
    if (typed) {
        if (!typed->dq || !typed->dk || !typed->dv) return HTREE_E_NULL;
        if (!aligned16(typed->dq) || !aligned16(typed->dk) || !aligned16(typed->dv)) return HTREE_E_ALIGN;
    } else if (!dq) {
        return HTREE_E_NULL;
    }
    // a query window is one part of a backward that the caller runs window by window over the same accumulators: only
    // meaningful with the flags that say which part it is
    const bool windowed = shape->T_q != 0 && (shape->T_q != shape->T || shape->t_offset != 0);
    if (windowed && !(flags & (HTREE_BWD_KEEP_ACCUM | HTREE_BWD_NO_FOLD))) return HTREE_E_WINDOW;
    AttnParams p;
    int rc = fill_params(p, shape, L, ln, q, layers_k, layers_v, cos_cache, sin_cache, n_pos, scale, parents, status, flags);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    for (int l = 0; l < L; ++l) {
        if (!parents[l] || !dk_levels[l] || !dv_levels[l]) return HTREE_E_NULL;
        if (!aligned16(dk_levels[l]) || !aligned16(dv_levels[l])) return HTREE_E_ALIGN;
        p.dk[l] = dk_levels[l]; p.dv[l] = dv_levels[l];
    }
    p.out = const_cast<void*>(out); p.dO = dO; p.gmax = const_cast<float*>(gmax); p.gsum = const_cast<float*>(gsum);
    p.dq = typed ? nullptr : dq;
    p.dq_typed = typed ? typed->dq : nullptr;
    if (cos_half && sin_half && aligned32(cos_half) && aligned32(sin_half)) {
        p.cosh = static_cast<const __half*>(cos_half); p.sinh = static_cast<const __half*>(sin_half);
    }
    // choose the kernel before anything is queued: a shape that neither kernel takes is refused with nothing launched
    bool fast = layers_k_rot != nullptr && !(flags & HTREE_FWD_GENERIC);
    if (fast) {
        for (int l = 0; l < L; ++l) {
            if (!layers_k_rot[l] || !aligned32(layers_k_rot[l]) || !aligned32(layers_v[l])) fast = false;
            p.lkr[l] = layers_k_rot[l];
        }
        fast = fast && aligned32(q) && aligned32(dO) && aligned32(out) && aligned16(typed ? typed->dq : (void*)dq) &&
               aligned32(cos_cache) && aligned32(sin_cache) && bwd_mma_supported(p, shape->dtype);
    }
    if (!fast && !bwd_generic_supported(p, shape->dtype)) return HTREE_E_UNSUPPORTED;
    for (int l = 0; l < L && !(flags & HTREE_BWD_KEEP_ACCUM); ++l) {   // gradient accumulators start at zero (src/backward.py:979-981)
        const size_t rows = (size_t)shape->B * ln[l] * shape->H_kv;
        cudaError_t e = cudaMemsetAsync(dk_levels[l], 0, rows * shape->K * sizeof(float), st);
        if (e == cudaSuccess) e = cudaMemsetAsync(dv_levels[l], 0, rows * shape->V * sizeof(float), st);
        if (e != cudaSuccess) return (int)e;
    }
    rc = fast ? launch_bwd_mma(p, shape->dtype, st) : launch_bwd_generic(p, shape->dtype, st);
    if (rc || (flags & HTREE_BWD_NO_FOLD)) return rc;
    return launch_tree_backward(*shape, L, ln, dk_levels, dv_levels, st, typed ? typed->dk : nullptr, typed ? typed->dv : nullptr);
}

}  // extern "C"
