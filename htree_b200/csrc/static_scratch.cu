// htree_b200_backward_static_scratch: the backward for callers that cannot hand the library any scratch memory.
//
// htree_b200_backward needs fp32 gradient accumulators for every pooled tree level (dk_levels[l], dv_levels[l] with
// l >= 1) next to its real outputs dq, dk, dv.  Some callers have no way to provide them: a host program that binds
// this library over a plain FFI and owns only the tensors its framework gave it has no device allocator of its own,
// and a process whose device memory is entirely reserved by its framework's pool (or that must not take the
// device-wide synchronisation an allocation or a free implies while other streams are busy) may not call cudaMalloc
// at that point.  This variant keeps the pooled-level accumulators in a fixed array that is part of the library image
// and lives in the memory of every GPU that loads the library until the process exits.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kScratchFloats = size_t(4) << 20;   // 4 Mi floats = 16 MiB per device
static __device__ __align__(256) float g_level_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of g_level_scratch on the CURRENT device.  In host code the array's name is only a handle of the
// symbol, not an address a kernel could use; the runtime resolves it per device.
int scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return HTREE_E_NODEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_level_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_ptr[dev] = static_cast<float*>(ptr);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" {

size_t htree_b200_static_scratch_bytes(void) { return kScratchFloats * sizeof(float); }

int htree_b200_backward_static_scratch(const HtreeShape* shape, const void* q, void* const* layers_k,
                                       void* const* layers_v, void* const* layers_k_rot, const float* cos_cache,
                                       const float* sin_cache, const void* cos_half, const void* sin_half,
                                       int32_t n_pos, float scale, const void* out,
                                       const void* dO, const float* gmax, const float* gsum, int32_t* const* parents,
                                       float* dq, float* dk, float* dv, int32_t* status, uint32_t flags, void* stream) {
    if (!shape || !dk || !dv) return HTREE_E_NULL;
    int32_t ln[HTREE_MAX_LEVELS];
    const int L = htree_b200_level_sizes(shape->T, shape->compression_rate, shape->max_top_nodes, ln, HTREE_MAX_LEVELS);
    if (L < 0) return L;
    if (shape->B <= 0 || shape->H_kv <= 0 || shape->K <= 0 || shape->V <= 0) return HTREE_E_SHAPE;
    // pooled levels, K part then V part of each level, every slice a multiple of 64 floats (256 bytes)
    size_t need = 0;
    size_t off_k[HTREE_MAX_LEVELS] = {}, off_v[HTREE_MAX_LEVELS] = {};
    for (int l = 1; l < L; ++l) {
        const size_t rows = (size_t)shape->B * ln[l] * shape->H_kv;
        off_k[l] = need; need += (rows * shape->K + 63) & ~size_t(63);
        off_v[l] = need; need += (rows * shape->V + 63) & ~size_t(63);
    }
    if (need > kScratchFloats) return HTREE_E_SCRATCH;
    float* base = nullptr;
    if (need) {
        const int rc = scratch_address(&base);
        if (rc) return rc;
    }
    float* dk_levels[HTREE_MAX_LEVELS] = {};
    float* dv_levels[HTREE_MAX_LEVELS] = {};
    dk_levels[0] = dk; dv_levels[0] = dv;
    for (int l = 1; l < L; ++l) { dk_levels[l] = base + off_k[l]; dv_levels[l] = base + off_v[l]; }
    // htree_b200_backward zero-fills every level it is given before accumulating, so whatever an earlier call left in
    // the array is cleared on the caller's stream before this call's kernels touch it.
    return htree_b200_backward(shape, q, layers_k, layers_v, layers_k_rot, cos_cache, sin_cache, cos_half, sin_half, n_pos, scale, out, dO,
                               gmax, gsum, parents, dq, dk_levels, dv_levels, nullptr, status, flags, stream);
}

}  // extern "C"
