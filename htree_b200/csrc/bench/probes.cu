// Ceilings of the two memory paths the attention kernels live on, measured with the kernels' own access patterns.
// They are the denominators for "how close is the kernel to what the chip can do": neither path is HBM (the trees and
// the gradient accumulators are L2-resident) nor the tensor pipe.
//   gather     random 256-byte rows of a table read with 32-byte loads, 8 rows x 128 contiguous bytes per warp
//              instruction: the pattern in which fwd_mma_kernel / bwd_mma_kernel fetch K' and V rows
//   reduction  red.global.add.v4.f32 into random 512-byte rows, four whole 128-byte lines per warp instruction: the
//              pattern in which bwd_mma_kernel adds its dK' / dV tiles into the level buffers
// No counterpart in the reference.  These are measurement aids of the benchmark, not part of the operator: they are built
// into a library of their own (libhtree_b200_probes.so) and are not declared in the operator's C header.
#include "../mma_common.cuh"

namespace htree {

__device__ __forceinline__ uint32_t probe_hash(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
    return x;
}

__global__ void __launch_bounds__(256) probe_gather_kernel(const uint8_t* table, uint32_t nrows, int iters, uint32_t* sink) {
    const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    uint32_t acc = 0;
    for (int it = 0; it < iters; ++it) {
        uint32_t x[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // 8 rows per instruction (lane / 4), 32 bytes per lane, the two halves of a row in turn
            const uint32_t row = probe_hash(gw * 7919u + (uint32_t)(it * 2 + (u >> 1)) * 8u + (lane >> 2)) % nrows;
            ldg32_stream(table + (size_t)row * 256 + (u & 1) * 128 + (lane & 3) * 32, x[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc ^= x[u][i];
    }
    if (acc == 0x9e3779b9u) sink[0] = acc;   // keeps the loads alive; practically never taken
}

__global__ void __launch_bounds__(128) probe_reduction_kernel(float* buf, uint32_t nrows, int iters) {
    const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    for (int it = 0; it < iters; ++it) {
#pragma unroll 4
        for (int j = 0; j < 32; ++j) {   // instruction j: 4 rows (8 lanes each), quarter j % 4 of every row
            const uint32_t row = probe_hash(gw * 977u + (uint32_t)it * 32u + 4u * (j >> 2) + (lane >> 3)) % nrows;
            red_add_v4(buf + (size_t)row * 128 + 32 * (j & 3) + 4 * (lane & 7), 1.f, 2.f, 3.f, 4.f);
        }
    }
}

template <typename Launch>
static int time_launches(Launch&& launch, int reps, cudaStream_t st, float* ms_out) {
    cudaEvent_t a, b;
    cudaError_t e = cudaEventCreate(&a);
    if (e != cudaSuccess) return (int)e;
    e = cudaEventCreate(&b);
    if (e != cudaSuccess) { cudaEventDestroy(a); return (int)e; }
    launch();                       // warm-up: brings the table into L2
    cudaEventRecord(a, st);
    for (int i = 0; i < reps; ++i) launch();
    cudaEventRecord(b, st);
    e = cudaEventSynchronize(b);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
    if (e == cudaSuccess) e = cudaGetLastError();
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    *ms_out = ms / reps;
    return (int)e;
}

}  // namespace htree

extern "C" int htree_probe_gather(void* table, int64_t table_bytes, int32_t reps, float* gbs, void* stream) {
    using namespace htree;
    if (!table || !gbs) return HTREE_E_NULL;
    if (table_bytes < (int64_t)256 * 64 || table_bytes / 256 > 0x7fffffff || reps <= 0) return HTREE_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(table) & 31u) return HTREE_E_ALIGN;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int blocks = sms * 8, iters = 256;
    const uint32_t nrows = (uint32_t)(table_bytes / 256);
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* sink = reinterpret_cast<uint32_t*>(table);   // written only if the xor of everything read hits one value
    float ms = 0.f;
    const int rc = time_launches([&] { probe_gather_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(table), nrows, iters, sink); },
                                 reps, st, &ms);
    if (rc) return rc;
    *gbs = (float)((double)blocks * 8 * iters * 4 * 1024.0 / (ms * 1e-3) / 1e9);
    return 0;
}

extern "C" int htree_probe_reduction(float* buffer, int64_t buffer_bytes, int32_t reps, float* gbs, void* stream) {
    using namespace htree;
    if (!buffer || !gbs) return HTREE_E_NULL;
    if (buffer_bytes < (int64_t)512 * 64 || buffer_bytes / 512 > 0x7fffffff || reps <= 0) return HTREE_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(buffer) & 15u) return HTREE_E_ALIGN;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int blocks = sms * 2, iters = 200;
    const uint32_t nrows = (uint32_t)(buffer_bytes / 512);
    cudaStream_t st = (cudaStream_t)stream;
    float ms = 0.f;
    const int rc = time_launches([&] { probe_reduction_kernel<<<blocks, 128, 0, st>>>(buffer, nrows, iters); }, reps, st, &ms);
    if (rc) return rc;
    *gbs = (float)((double)blocks * 4 * iters * 16384.0 / (ms * 1e-3) / 1e9);
    return 0;
}
