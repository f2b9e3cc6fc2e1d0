// Tensor-core forward for 16-bit storage types: one WARP per (batch, query position, KV head) group, all tree levels
// in one launch, every operand moved global/L2 -> registers -> mma.sync (no shared-memory staging, no block barriers).
//
// Replaces the same reference kernels as the generic forward (htree_select_accumulate_gqa_kernel,
// htree_bottom_accumulate_gqa_kernel, htree_merge_to_global_kernel, htree_final_normalize_kernel;
// src/parallel.py:248-867) for bf16/fp16, head_dim 64 or 128, K == V, group size <= 16, compression_rate 16 or 8
// (with 8 children per parent the second score tile stays empty).
//
// Design notes
//  * M = the GQA group (<= 16 query heads) maps exactly onto the M = 16 rows of mma.sync.m16n8k16; candidates are the
//    N dimension of the score product and the K dimension of the P.V product, so a chunk of 16 candidates (= the
//    children of one parent) is two n8 score tiles and one k16 accumulation step.
//  * RoPE.  The reference rotates every gathered key by its position j in the query's candidate list
//    (src/parallel.py:687-692).  With j = 16*a + c (parent slot a, child index c) and rotations composing additively,
//        (R(p) q)^T (R(j) k) = (R(p - 16a) q)^T (R(c) k),
//    and c = node % 16 does not depend on the query.  The tree build therefore also stores K' = R(node % 16) K once
//    per level, and this kernel rotates the QUERY once per parent (by p - 16a) while keys go from memory straight
//    into B fragments.  Both operands see exactly one rounding, as in a direct evaluation; that rounding is to IEEE
//    half for every storage type (K' is stored as half, the rotated query is packed as half), because half's 11-bit
//    significand keeps the score noise 8x below bf16's and with it the rate of Top-K near-tie swaps.
//  * Fragments are loaded so that no data movement is needed: the contraction index of the score product is
//    permuted (thread r of a quad owns rotation pairs [P*r, P*(r+1)) of both halves), applied consistently to A and
//    B; the value rows are loaded as one 32-byte (D = 128) or 16-byte (D = 64) piece per row and thread and byte-permuted
//    into k-major B fragments.  Gathered rows are used once and are not allocated in L1.
//  * Upper levels run two passes over the candidates: pass 1 scores and stores only the shared importance
//    (4 bytes per candidate in shared memory), an exact Top-K (bitwise search for the K-th largest key, ties to the
//    smaller position, right-most forced) picks the kept set, pass 2 re-scores and accumulates the others.
//    The leaf level is a single pass.  One running (max, sum, out) state spans all levels, which is the same
//    softmax as the reference's per-level states merged afterwards (src/naive.py:215-223).
#include "mma_common.cuh"
#include "pipe.cuh"

namespace htree {

#ifdef HTREE_FWD_MAXNREG
#define HTREE_FWD_BOUNDS __maxnreg__(HTREE_FWD_MAXNREG)
#else
#define HTREE_FWD_BOUNDS __launch_bounds__(HTREE_FWD_WARPS * 32, HTREE_FWD_MIN_BLOCKS)
#endif
#ifndef HTREE_FWD_WARPS
#define HTREE_FWD_WARPS 4
#endif
constexpr int MW = HTREE_FWD_WARPS;   // warps (= queries) per block
#ifndef HTREE_FWD_MIN_BLOCKS
#define HTREE_FWD_MIN_BLOCKS 2   // register budget: 2 blocks of 128 threads per SM (255 registers)
#endif

struct MmaSmem {   // per warp
    float* imp;      // [maxc]   shared importance / its bit pattern
    float* cmax;     // [TK]     per-chunk score maximum
    uint32_t* selw;  // [maxc/32] kept-candidate bit mask
    int32_t* par;    // [2][TK]
};

#ifndef HTREE_SEL_MIN_BLOCKS
#define HTREE_SEL_MIN_BLOCKS 4   // the selection kernel carries no accumulators: 128 registers, 16 warps per SM
#endif
// Shared memory of one warp: the selection scratch (importance per candidate, per-chunk maxima; not needed by the
// accumulation kernel), the kept-candidate bit mask and two parent lists, rounded up to 128 bytes; `pipe_bytes` more for
// the operand ring of the pipelined kernels.
__host__ __device__ inline size_t mma_smem_per_warp(int TK, int CR, bool selection_scratch = true, size_t pipe_bytes = 0) {
    const size_t maxc = (size_t)TK * CR;
    size_t b = sizeof(uint32_t) * ((maxc + 31) / 32) + sizeof(int32_t) * 2 * TK;
    if (selection_scratch) b += sizeof(float) * maxc + sizeof(float) * TK;
    b = (b + 127) & ~size_t(127);
    return b + pipe_bytes;
}

// Pipelined kernels (128-wide heads, 16 children per parent, 16-bit types; selection kernel and accumulation kernel): what
// a chunk needs - the parent's blocked keys (4 KB), when accumulating its blocked values (4 KB), and the rows of the rotary
// tables for the chunk's rotation - arrives in a per-warp ring in shared memory by asynchronous bulk copies that the warp
// itself issues a few chunks ahead, each completing on the slot's mbarrier; fragments are then read with conflict-free
// 16-byte shared loads right before the MMAs that consume them.  Against gathering into registers this keeps loads in
// flight without holding registers for them, and takes the L2 latency of keys, values AND table rows (the tables do not
// stay in what is left of L1) off the start of every chunk's dependency chain.
#ifndef HTREE_PIPE_STAGES_SEL
#define HTREE_PIPE_STAGES_SEL 2
#endif
#ifndef HTREE_PIPE_STAGES_ACC
#define HTREE_PIPE_STAGES_ACC 2
#endif
#ifndef HTREE_PIPE_SEL_WARPS
#define HTREE_PIPE_SEL_WARPS 5      // selection kernel: 3 blocks of 5 warps per SM (the ring costs shared memory)
#endif
#ifndef HTREE_PIPE_SEL_BLOCKS
#define HTREE_PIPE_SEL_BLOCKS 3
#endif
#ifndef HTREE_PIPE_ACC_WARPS
#define HTREE_PIPE_ACC_WARPS 3      // accumulation kernel, groups of at most 8 heads: 3 blocks of 3 warps per SM (227 registers)
#endif
#ifndef HTREE_PIPE_ACC_WARPS_G16
#define HTREE_PIPE_ACC_WARPS_G16 4  // groups of 9..16 heads: 3 blocks of 4 warps (168 registers, 12 bytes of spills)
#endif
#ifndef HTREE_PIPE_ACC_BLOCKS
#define HTREE_PIPE_ACC_BLOCKS 3
#endif
constexpr int kPipeWaitCap = 1 << 16;   // attempts per wait before the kernel gives up and reports status bit 16
// bytes of one ring slot: blocked keys, blocked values (accumulation), table rows (fp32 cos + sin: 2 * 256 bytes where the
// query is rotated in fp32 - always in the selection kernel -, packed-half cos + sin: 2 * 128 bytes otherwise)
__host__ __device__ constexpr uint32_t pipe_slot_bytes(int mode, bool rot16) {
    return (mode == 1 ? 4096u : 8192u) + ((mode == 1 || !rot16) ? 512u : 256u);
}
__host__ __device__ constexpr size_t pipe_bytes_per_warp(int mode, bool rot16) {
    return (size_t)(mode == 1 ? HTREE_PIPE_STAGES_SEL : HTREE_PIPE_STAGES_ACC) * pipe_slot_bytes(mode, rot16) + 128;
}
#ifndef HTREE_SEL_WARPS
#define HTREE_SEL_WARPS HTREE_FWD_WARPS
#endif
// Measured on B200, cfg3 (B=4, T=65536, H=64, H_kv=4, D=128, bf16), ms per launch: selection kernel 56.20 gathering into
// registers (4 blocks x 4 warps) vs 56.27 pipelined (3 x 5 warps) vs 59.2 (2 x 7); accumulation kernel 107.2 gathering
// (2 x 4 warps) / 104.2 (3 x 3) vs pipelined 117.7 (2 x 4, 3 stages) / 102.8 (3 x 3, 2 stages) / 117.7 (4 x 2).  Neither
// kernel is bound by the latency of its gathers: the selection kernel keeps its register path (more resident warps, no
// ring), the accumulation kernel takes the pipelined one, whose short-lived operand registers also make 12 warps per SM
// possible (the register path spilled there): whole forward, pipelined accumulation at 3 x 3 / 3 x 4 / 2 x 6 / 4 x 3 warps:
// cfg3 (groups of 16 heads) 158.8 / 154.5 / 155.6 / 155.5 ms, cfg4 (groups of 8) 399.8 / 403.0 / 403.7 / 404.4 ms.
#ifndef HTREE_PIPE_SEL
#define HTREE_PIPE_SEL 0     // 1: the selection kernel streams its operands too
#endif
#ifndef HTREE_PIPE_ACC
#define HTREE_PIPE_ACC 1     // 0: the accumulation kernel always gathers into registers
#endif
__host__ __device__ constexpr int fwd_warps_per_block(int mode, bool pipe, int nr = 1) {
    return pipe ? (mode == 1 ? HTREE_PIPE_SEL_WARPS : (nr == 2 ? HTREE_PIPE_ACC_WARPS_G16 : HTREE_PIPE_ACC_WARPS))
                : (mode == 1 ? HTREE_SEL_WARPS : HTREE_FWD_WARPS);
}
// Selection kernel for groups of 9..16 heads: 3 blocks of 4 warps (152 registers, nothing spilled) measured 49.2 ms against
// 50.5 ms for 4 blocks (128 registers, the raw query rows spilled and re-read from local memory in every chunk: two thirds
// of that kernel's L1 wavefronts); groups of at most 8 heads fit 128 registers and keep 4 blocks (cfg4: 140 against 152 ms).
__host__ __device__ constexpr int fwd_blocks_per_sm(int mode, bool pipe, bool x3, int nr = 1, int d = 64) {
    return pipe ? (mode == 1 ? HTREE_PIPE_SEL_BLOCKS : HTREE_PIPE_ACC_BLOCKS)
                : (mode == 1 ? ((x3 || (nr == 2 && d == 128)) ? 3 : HTREE_SEL_MIN_BLOCKS) : HTREE_FWD_MIN_BLOCKS);
}

// MODE 0: whole forward in one kernel.  MODE 1: selections only (no accumulator state, so far fewer registers and more
// resident warps); MODE 2: accumulation only, reading the per-level parent lists that a MODE 1 launch wrote.  When the
// caller provides parent buffers the forward runs as MODE 1 + MODE 2.
// NR = 1: groups of at most 8 heads (rows g+8 of every fragment are padding and their ALU work is skipped).
// T = float: split-half products (mma_common.cuh), 64-wide heads; K' and the blocked values then hold a hi and a lo plane.
template <typename T, int D, bool ROT16, int MODE, int NR, int CR, bool PIPE = false>
__global__ void __launch_bounds__(fwd_warps_per_block(MODE, PIPE, NR) * 32, fwd_blocks_per_sm(MODE, PIPE, std::is_same<T, float>::value, NR, D))
fwd_mma_kernel(const __grid_constant__ AttnParams p) {
    constexpr bool X3 = std::is_same<T, float>::value;
    constexpr int MWK = fwd_warps_per_block(MODE, PIPE, NR);   // warps (= queries) per block
    static_assert(!PIPE || (D == 128 && CR == 16 && !X3 && (MODE == 1 || MODE == 2)), "pipelined kernels: 128-wide heads, 16 children, 16-bit types");
    constexpr bool FRAGV = kFragmentMajor<D, CR, X3>;   // element order of the blocked values
    constexpr uint32_t kAllChildren = (1u << CR) - 1u;   // CR = children per parent: 16, or 8 (then tile 1 stays empty)
    constexpr int HALF = D / 2;
    constexpr int KS = D / 16;        // k-steps of the score product
    constexpr int PPT = HALF / 4;     // rotation pairs owned by one thread of a quad
    constexpr int NV = PPT / 8;       // 16-byte loads per (row, half): 2 for D=128, 1 for D=64
    constexpr int VB = D / 8;         // value columns one thread loads per row: one 32-byte (D=128) or 16-byte (D=64) piece
    constexpr int NOT = D / 8;        // n8 output tiles
    using F = Frag<typename std::conditional<X3, __half, T>::type>;   // P.V product: values stay in their storage type (fp32: half planes)
    using FS = Frag<__half>;    // score product: rotated queries and K' are IEEE half for every storage type
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, r = lane & 3;
    const int tl = blockIdx.x * MWK + warp;
    if (tl >= p.Tq) return;                        // warps are independent: only __syncwarp below
    const int t = p.t0 + tl;
    const int b = blockIdx.y / p.Hkv, hk = blockIdx.y % p.Hkv;
    const int G = p.G, TK = p.TK, L = p.L;
    const int maxc = TK * CR;
    constexpr bool kScratch = MODE != 2;           // the accumulation kernel keeps no importance array
    unsigned char* wbase = smem_raw + (size_t)warp * mma_smem_per_warp(TK, CR, kScratch, PIPE ? pipe_bytes_per_warp(MODE, ROT16) : 0);
    float* imp = reinterpret_cast<float*>(wbase);
    float* cmax = imp + (kScratch ? maxc : 0);
    uint32_t* selw = reinterpret_cast<uint32_t*>(cmax + (kScratch ? TK : 0));
    int32_t* par = reinterpret_cast<int32_t*>(selw + (maxc + 31) / 32);
    int32_t* nxt = par + TK;

    // ---- operand ring of the pipelined kernels ----
    constexpr int NSTG = MODE == 1 ? HTREE_PIPE_STAGES_SEL : HTREE_PIPE_STAGES_ACC;
    constexpr uint32_t SLOT = pipe_slot_bytes(MODE, ROT16);
    constexpr uint32_t TAB_OFF = MODE == 1 ? 4096u : 8192u;                 // table rows follow the operand blocks
    constexpr bool kTabF32 = MODE == 1 || !ROT16;                           // fp32 rows (256 B each) or packed-half rows (128 B each)
    constexpr uint32_t TAB_ROW = kTabF32 ? 256u : 128u;
    unsigned char* ring = wbase + mma_smem_per_warp(TK, CR, kScratch);      // 128-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)NSTG * SLOT);
    uint32_t pn = 0, pissued = 0;     // chunks consumed / issued by this warp so far: slot = n % NSTG, phase parity = (n / NSTG) & 1
    const unsigned char* kblk = nullptr;    // this level's blocked keys / values of (b, hk); parents are blk_stride bytes apart
    const unsigned char* vblk = nullptr;
    int64_t blk_stride = 0;
    [[maybe_unused]] int pipe_level = 0;
    int blk_count = 0, pipe_rp = 0;         // pipe_rp: rotation position of the level (the chunk at slot a rotates by rp - CR*a)
    if constexpr (PIPE) {
        if (lane == 0) {
            for (int i = 0; i < NSTG; ++i) mbar_init(&bars[i], 1);
            fence_barrier_init();
        }
#ifdef HTREE_FWD_KNOCK_ALLCOPY
        for (uint32_t i = lane * 16u; i < (uint32_t)NSTG * SLOT; i += 512u) *reinterpret_cast<uint4*>(ring + i) = make_uint4(0u, 0u, 0u, 0u);
#endif
        __syncwarp();
    }
    auto pipe_issue = [&](uint32_t n, int a) {       // lane 0: start the copies for the chunk at parent slot a into ring slot n % NSTG
        int pb = par[a];
        if (pb < 0 || pb >= blk_count) pb = 0;       // flagged where the chunk is consumed
        const int sl = (int)(n % NSTG);
        unsigned char* dst = ring + (size_t)sl * SLOT;
#ifdef HTREE_FWD_KNOCK_ALLCOPY   // timing experiments only: no copies and no waits, the kernels compute on a zero-filled ring
        return;
#endif
#ifdef HTREE_FWD_KNOCK_KCOPY   // timing experiments only: upper-level chunks of the accumulation kernel bring their values alone
        if (MODE == 2 && pipe_level > 0) {
            mbar_arrive_expect_tx(&bars[sl], 4096u);
            bulk_copy_g2s(dst + 4096, vblk + (int64_t)pb * blk_stride, 4096u, &bars[sl]);
            return;
        }
#endif
        mbar_arrive_expect_tx(&bars[sl], SLOT);
        bulk_copy_g2s(dst, kblk + (int64_t)pb * blk_stride, 4096u, &bars[sl]);
        if (MODE == 2) bulk_copy_g2s(dst + 4096, vblk + (int64_t)pb * blk_stride, 4096u, &bars[sl]);
        const int64_t row = (int64_t)(pipe_rp - CR * a);
        if (kTabF32) {
            bulk_copy_g2s(dst + TAB_OFF, p.cosc + row * HALF, TAB_ROW, &bars[sl]);
            bulk_copy_g2s(dst + TAB_OFF + TAB_ROW, p.sinc + row * HALF, TAB_ROW, &bars[sl]);
        } else {
            bulk_copy_g2s(dst + TAB_OFF, p.cosh + row * HALF, TAB_ROW, &bars[sl]);
            bulk_copy_g2s(dst + TAB_OFF + TAB_ROW, p.sinh + row * HALF, TAB_ROW, &bars[sl]);
        }
    };
    // Give up after a wait ran out: flag it, wait (bounded again) for the copies still in flight into this warp's ring, and
    // leave.  Never taken unless something is badly wrong; it keeps the kernel from spinning forever.
    auto pipe_abort = [&]() {
        if (lane == 0 && p.status) atomicOr(p.status, 16);
        for (uint32_t n = pn; n < pissued; ++n) mbar_wait_bounded(&bars[n % NSTG], (n / NSTG) & 1u, kPipeWaitCap);
    };
    // before the first chunk of a loop over `count` parents (par[0 .. count)): fill the ring
    auto pipe_begin = [&](int count) {
        __syncwarp();
        const int ahead = count < NSTG - 1 ? count : NSTG - 1;
        if (lane == 0) {
            fence_proxy_async();
            for (int j = 0; j < ahead; ++j) pipe_issue(pn + j, j);
        }
        pissued = pn + ahead;
    };
    // chunk a of `count`: refill the slot the previous chunk used, then wait for this chunk's block(s).  Returns the slot,
    // or nullptr after a wait ran out (the caller returns).
    auto pipe_next = [&](int a, int count) -> const unsigned char* {
        __syncwarp();                                   // every lane is done reading the slot that is refilled now
        if (a + NSTG - 1 < count) {
            if (lane == 0) { fence_proxy_async(); pipe_issue(pn + NSTG - 1, a + NSTG - 1); }
            pissued = pn + NSTG;
        }
        const int sl = (int)(pn % NSTG);
#ifndef HTREE_FWD_KNOCK_ALLCOPY
        if (!mbar_wait_bounded(&bars[sl], (pn / NSTG) & 1u, kPipeWaitCap)) { pipe_abort(); return nullptr; }
#endif
        ++pn;
        return ring + (size_t)sl * SLOT;
    };
    const unsigned char* slot = nullptr;                // operand blocks of the chunk being computed

    constexpr bool kSelectKernel = MODE == 1, kAccumulateKernel = MODE == 2;
    const bool select_only = kSelectKernel || (MODE == 0 && (p.flags & HTREE_FWD_SELECT_ONLY) != 0);
    const int64_t hbase = ((int64_t)b * p.Tq + tl) * p.H + (int64_t)hk * G;
    const int64_t qidx = ((int64_t)b * p.Tq + tl) * p.Hkv + hk;
    const bool row_ok[2] = {g < G, NR == 2 && g + 8 < G};

    // raw queries of rows g and g+8: pairs [PPT*r, PPT*(r+1)) of the low and of the high half
    uint32_t qraw[2][2][X3 ? 2 * KS : KS];     // 16-bit types: IEEE half pairs; fp32: the float bits
    if constexpr (X3) load_rows_f32<D>(reinterpret_cast<const float*>(p.q) + hbase * D, g, r, row_ok, qraw);
    else load_rows_half<T, D>(reinterpret_cast<const T*>(p.q) + hbase * D, g, r, row_ok, qraw);
    constexpr bool rot16 = ROT16;   // packed-half rotation where the Top-K is not being decided

    float O[NOT][4];
#pragma unroll
    for (int i = 0; i < NOT; ++i) { O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f; }
    // Online softmax with a lazily updated reference: probabilities are taken relative to m_run, which is only moved (and
    // the accumulators rescaled) when a row maximum exceeds it by more than kLazyMax, so exp(s - m_run) <= e^kLazyMax; the
    // true running maximum is tracked separately for the (gmax, gsum) the backward reads.  With 16 heads sharing a warp
    // an exact running maximum would move in most chunks and cost 64 multiplies each time.
    constexpr float kLazyMax = 8.f;
    float m_run[2] = {-1.0e30f, -1.0e30f}, m_true[2] = {-1.0e30f, -1.0e30f}, s_run[2] = {0.f, 0.f};
    float m_run2[2] = {-1.0e30f * kLog2e, -1.0e30f * kLog2e};      // m_run in units of log 2, the form the exponentials take

    {   // virtual parents of the top level (src/parallel.py:1026-1038)
        int np0 = (int)(((int64_t)t / p.lpow[L - 1]) / CR) + 1;
        if (np0 > TK) np0 = TK;
        for (int i = lane; i < TK; i += 32) par[i] = i < np0 ? i : -1;
    }
    __syncwarp();

    for (int l = L - 1; l >= 0; --l) {
        const int Nl = p.ln[l];
        const __half* lkr = reinterpret_cast<const __half*>(p.lkr[l]);
        if (kAccumulateKernel) {
            __syncwarp();
            for (int i = lane; i < TK; i += 32) par[i] = load_parent(p, l, qidx * TK + i);
            __syncwarp();
        } else if (p.parents[l]) {
            for (int i = lane; i < TK; i += 32) store_parent(p, l, qidx * TK + i, par[i]);
        }
        if (select_only && l == 0) break;
        int np = 0;
        for (int i = lane; i < TK; i += 32) np += par[i] >= 0;
        np = __reduce_add_sync(0xffffffffu, np);
        const int rc = (int)(((int64_t)t / p.lpow[l]) % CR);
        const int nc = (np - 1) * CR + rc + 1, rp = nc - 1;

        // S0/S1 = scores of the 16 children of parent slot `a` against the 16 query rows.  `select` = this pass
        // decides the Top-K: the query is then always rotated in fp32.
        // per-lane bases into this level: only node * rstride is left to add per chunk
        const int rstride = p.Hkv * D;
        // a gathered row is used once and is not allocated in L1; the selection kernel, where the top level is a larger
        // share of the rows, keeps that level (shared by neighbouring queries, small enough to live in L1) cached
        const bool stream_rows = kSelectKernel ? l < L - 1 : true;
        const __half* kq = lkr + ((int64_t)b * Nl * p.Hkv + hk) * D + (D == 64 ? D / 4 : D / 8) * r;
        // blocked values of this level: block (b, parent, hk) holds CR*D elements, lane (g, r) owns words [(8r+g)*CHW, +CHW)
        const int64_t vb_stride = (int64_t)p.Hkv * (CR * D / 2);     // 32-bit words between consecutive parents
        const int64_t vb_plane = (int64_t)p.B * ((Nl + CR - 1) / CR) * vb_stride;   // fp32 storage: words from the hi plane to the lo plane
        const uint32_t* vbq = reinterpret_cast<const uint32_t*>(p.lvb[l]) +
                              ((int64_t)b * ((Nl + CR - 1) / CR) * p.Hkv + hk) * (CR * D / 2) +
                              (FRAGV ? 4 * lane : (8 * r + g) * (NOT * (CR / 8)));
        if constexpr (PIPE) {
            blk_count = (Nl + CR - 1) / CR;
            blk_stride = (int64_t)p.Hkv * (CR * D * 2);
            pipe_rp = rp; pipe_level = l;
            kblk = reinterpret_cast<const unsigned char*>(p.lkb[l]) + ((int64_t)b * blk_count * p.Hkv + hk) * (CR * D * 2);
            vblk = reinterpret_cast<const unsigned char*>(p.lvb[l]) + ((int64_t)b * blk_count * p.Hkv + hk) * (CR * D * 2);
        }
        auto score = [&](int a, float (&S0)[4], float (&S1)[4], bool select) {
            int node0 = par[a] * CR;
            if (node0 < 0 || node0 >= Nl) { if (p.status) atomicOr(p.status, 4); node0 = 0; }
#ifdef HTREE_FWD_KNOCK_SCORE   // timing experiments only: levels in the kernel's bit mask (selection kernel: bits 0-7,
            // accumulation kernel: bits 8-15) are not scored; results are wrong
            if (((kAccumulateKernel ? (HTREE_FWD_KNOCK_SCORE) >> 8 : (HTREE_FWD_KNOCK_SCORE)) >> l) & 1) {
                S0[0] = S0[1] = S0[2] = S0[3] = S1[0] = S1[1] = S1[2] = S1[3] = 0.f;
                return;
            }
#endif
            if constexpr (PIPE) {
                // the rotation of a chunk is fixed by the kernel: fp32 tables where the Top-K is decided (selection kernel) or
                // no packed-half tables were given, packed-half tables otherwise; its table rows are in the slot
                score_chunk_sm<D, !kTabF32, NR>(p, reinterpret_cast<const uint4*>(slot), slot + TAB_OFF, lane, qraw, S0, S1);
                return;
            }
            if constexpr (X3) {
                score_chunk_x3<D, NR, CR>(p, kq, (int64_t)p.B * Nl * rstride, rstride, Nl, node0, rp - CR * a, g, r, qraw, S0, S1, stream_rows);
            } else {
                uint32_t unused[1][4];
                if (rot16 && !select) score_chunk<D, false, true, false, NR, CR>(p, kq, rstride, Nl, node0, rp - CR * a, g, r, qraw, S0, S1, unused, nullptr, stream_rows);
                else score_chunk<D, false, false, false, NR, CR>(p, kq, rstride, Nl, node0, rp - CR * a, g, r, qraw, S0, S1, unused, nullptr, stream_rows);
            }
        };

        // online-softmax accumulation of the columns in `mask` (bit c = child c of the parent at slot a)
        auto accumulate_chunk = [&](int a, float (&S0)[4], float (&S1)[4], uint32_t mask) {
            int pblk = par[a];
            if (pblk < 0 || (int64_t)pblk * CR >= Nl) pblk = 0;
            const int col[4] = {2 * r, 2 * r + 1, 8 + 2 * r, 9 + 2 * r};
            const bool cv[4] = {(mask >> col[0] & 1) != 0, (mask >> col[1] & 1) != 0, (mask >> col[2] & 1) != 0, (mask >> col[3] & 1) != 0};
            // value fragments first (longest latency): this lane's piece of the parent's blocked values, NOT*NB words
            // that ARE the B fragments of the P.V products; the warp reads the block front to back
            constexpr int NB = CR / 8, CHW = NOT * NB;
            uint32_t vw[CHW], vl[X3 ? CHW : 1];     // fp32 storage: hi plane and lo plane
            if constexpr (PIPE) {
                // piece i of this lane = the fragments of output tiles 2i and 2i+1, read from the chunk's slot
                const uint4* vs = reinterpret_cast<const uint4*>(slot + 4096);
#pragma unroll
                for (int i = 0; i < CHW / 4; ++i) {
                    const uint4 x = lds128(vs + i * 32 + lane);
                    vw[4 * i] = x.x; vw[4 * i + 1] = x.y; vw[4 * i + 2] = x.z; vw[4 * i + 3] = x.w;
                }
            } else if constexpr (FRAGV) {
                // fragment-major blocks read straight from global memory (the one-kernel forward): 16-byte pieces
                const uint4* src = reinterpret_cast<const uint4*>(vbq + (int64_t)pblk * vb_stride);
#pragma unroll
                for (int i = 0; i < CHW / 4; ++i) {
                    const uint4 x = stream_rows ? ldg16_stream(src + i * 32) : ldg16(src + i * 32);
                    vw[4 * i] = x.x; vw[4 * i + 1] = x.y; vw[4 * i + 2] = x.z; vw[4 * i + 3] = x.w;
                }
            } else {
                const uint32_t* src = vbq + (int64_t)pblk * vb_stride;
#pragma unroll
                for (int i = 0; i < CHW / 8; ++i) {
                    uint32_t t8[8];
                    if (stream_rows) ldg32_stream(src + 8 * i, t8); else ldg32(src + 8 * i, t8);
#pragma unroll
                    for (int u = 0; u < 8; ++u) vw[8 * i + u] = t8[u];
                    if constexpr (X3) {
                        if (stream_rows) ldg32_stream(src + vb_plane + 8 * i, t8); else ldg32(src + vb_plane + 8 * i, t8);
#pragma unroll
                        for (int u = 0; u < 8; ++u) vl[8 * i + u] = t8[u];
                    }
                }
            }
            const float NINF = -INFINITY;
            float s[2][4];   // [row][tile0 c0, tile0 c1, tile1 c0, tile1 c1]
            s[0][0] = (cv[0] && row_ok[0]) ? S0[0] : NINF; s[0][1] = (cv[1] && row_ok[0]) ? S0[1] : NINF;
            s[0][2] = (cv[2] && row_ok[0]) ? S1[0] : NINF; s[0][3] = (cv[3] && row_ok[0]) ? S1[1] : NINF;
            s[1][0] = (cv[0] && row_ok[1]) ? S0[2] : NINF; s[1][1] = (cv[1] && row_ok[1]) ? S0[3] : NINF;
            s[1][2] = (cv[2] && row_ok[1]) ? S1[2] : NINF; s[1][3] = (cv[3] && row_ok[1]) ? S1[3] : NINF;
            float mr[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                float m = fmaxf(fmaxf(s[rr][0], s[rr][1]), fmaxf(s[rr][2], s[rr][3]));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));     // (a quad-masked redux.sync measured far slower than the two
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));     // shuffles: 176 ms against 98 ms per launch)
                mr[rr] = m;
            }
            m_true[0] = fmaxf(m_true[0], mr[0]); m_true[1] = fmaxf(m_true[1], mr[1]);
            if (__any_sync(0xffffffffu, mr[0] > m_run[0] + kLazyMax || mr[1] > m_run[1] + kLazyMax)) {
                const float n0 = fmaxf(m_run[0], mr[0]), n1 = fmaxf(m_run[1], mr[1]);
                const float a0 = X3 ? __expf(m_run[0] - n0) : ex2_approx(m_run2[0] - n0 * kLog2e);
                const float a1 = X3 ? __expf(m_run[1] - n1) : ex2_approx(m_run2[1] - n1 * kLog2e);
                m_run[0] = n0; m_run[1] = n1;
                m_run2[0] = n0 * kLog2e; m_run2[1] = n1 * kLog2e;
                s_run[0] *= a0; s_run[1] *= a1;
#pragma unroll
                for (int i = 0; i < NOT; ++i) {
                    O[i][0] *= a0; O[i][1] *= a0;
                    if (NR == 2) { O[i][2] *= a1; O[i][3] *= a1; }
                }
            }
            float pr[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int rr = 0; rr < NR; ++rr)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    // exp(s - m_run); 16-bit storage: one multiply-add and the hardware 2^x against the reference kept in
                    // units of log 2 (its rounding, 1e-6 relative, is common to a row but not to a re-based sum: fp32 storage
                    // keeps the plain form)
                    pr[rr][c] = X3 ? __expf(s[rr][c] - m_run[rr]) : ex2_approx(fmaf(s[rr][c], kLog2e, -m_run2[rr]));
                    s_run[rr] += pr[rr][c];
                }
            // output tile w, column c <-> value column VB*c + w (the blocked layout is built for exactly this mapping);
            // children that are not accumulated have probability 0, and every value of the block is finite
            if constexpr (X3) {
                uint32_t ph[4], pl[4];
                split_half2(pr[0][0], pr[0][1], ph[0], pl[0]); split_half2(pr[1][0], pr[1][1], ph[1], pl[1]);
                split_half2(pr[0][2], pr[0][3], ph[2], pl[2]); split_half2(pr[1][2], pr[1][3], ph[3], pl[3]);
                // The chunk's three products are summed from zero and then added to the running output with an ordinary
                // (round-to-nearest) fp32 add: the tensor core's own accumulation truncates, and over the ~10^3 chunks of a
                // query that bias would reach 1e-4 relative.
#pragma unroll
                for (int w = 0; w < NOT; ++w) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    F::mma(acc, pl[0], pl[1], pl[2], pl[3], vw[w * NB], NB == 2 ? vw[w * NB + 1] : 0u);
                    F::mma(acc, ph[0], ph[1], ph[2], ph[3], vl[w * NB], NB == 2 ? vl[w * NB + 1] : 0u);
                    F::mma(acc, ph[0], ph[1], ph[2], ph[3], vw[w * NB], NB == 2 ? vw[w * NB + 1] : 0u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) O[w][i] += acc[i];
                }
            } else {
                const uint32_t pa0 = F::pack(pr[0][0], pr[0][1]), pa1 = F::pack(pr[1][0], pr[1][1]);
                const uint32_t pa2 = F::pack(pr[0][2], pr[0][3]), pa3 = F::pack(pr[1][2], pr[1][3]);
#pragma unroll
                for (int w = 0; w < NOT; ++w) F::mma(O[w], pa0, pa1, pa2, pa3, vw[w * NB], NB == 2 ? vw[w * NB + 1] : 0u);
            }
        };

        if (l > 0 && kAccumulateKernel) {
#ifdef HTREE_FWD_KNOCK_LEVEL   // timing experiments only: the accumulation kernel leaves out the levels of this bit mask
            if (((HTREE_FWD_KNOCK_LEVEL) >> l) & 1) continue;
#endif
            if (nc > TK) {
                // kept-candidate bit mask from the two sorted lists: the level's parents and the next level's parents
                for (int i = lane; i < (nc + 31) / 32; i += 32) selw[i] = 0u;
                for (int i = lane; i < TK; i += 32) nxt[i] = load_parent(p, l - 1, qidx * TK + i);
                __syncwarp();
                for (int i = lane; i < TK; i += 32) {
                    const int node = nxt[i];
                    if (node < 0) continue;
                    const int parent = node / CR;
                    int lo = 0, hi = np;
                    while (lo < hi) { const int mid = (lo + hi) >> 1; if (par[mid] < parent) lo = mid + 1; else hi = mid; }
                    if (lo < np && par[lo] == parent) {
                        const int j = lo * CR + node % CR;
                        atomicOr(&selw[j >> 5], 1u << (j & 31));
                    }
                }
                __syncwarp();
                if constexpr (PIPE) pipe_begin(np);
                for (int a = 0; a < np; ++a) {
                    if constexpr (PIPE) { slot = pipe_next(a, np); if (!slot) return; }
                    const uint32_t kept = (selw[(a * CR) >> 5] >> ((a * CR) & 31)) & kAllChildren;
                    const uint32_t valid = a == np - 1 ? ((2u << rc) - 1u) : kAllChildren;
                    const uint32_t mask = ~kept & valid;
                    if (mask == 0) continue;
                    float S0[4], S1[4];
                    score(a, S0, S1, false);
                    accumulate_chunk(a, S0, S1, mask);
                }
            }
        } else if (l > 0) {
            if (nc <= TK) {   // every candidate is kept, nothing to score or accumulate
                __syncwarp();
                for (int j = lane; j < TK; j += 32) nxt[j] = j < nc ? par[j / CR] * CR + j % CR : -1;
            } else {
                // ---- pass 1: shared importance of every candidate ----
                if constexpr (PIPE) pipe_begin(np);
                for (int a = 0; a < np; ++a) {
                    if constexpr (PIPE) { slot = pipe_next(a, np); if (!slot) return; }
                    float S0[4], S1[4];
                    score(a, S0, S1, true);
                    const int jb = a * CR;
                    const bool cv[4] = {jb + 2 * r < nc, jb + 2 * r + 1 < nc, CR > 8 && jb + 8 + 2 * r < nc, CR > 8 && jb + 9 + 2 * r < nc};
                    const float NINF = -INFINITY;
                    float s[2][4];
                    s[0][0] = (cv[0] && row_ok[0]) ? S0[0] : NINF; s[0][1] = (cv[1] && row_ok[0]) ? S0[1] : NINF;
                    s[0][2] = (cv[2] && row_ok[0]) ? S1[0] : NINF; s[0][3] = (cv[3] && row_ok[0]) ? S1[1] : NINF;
                    s[1][0] = (cv[0] && row_ok[1]) ? S0[2] : NINF; s[1][1] = (cv[1] && row_ok[1]) ? S0[3] : NINF;
                    s[1][2] = (cv[2] && row_ok[1]) ? S1[2] : NINF; s[1][3] = (cv[3] && row_ok[1]) ? S1[3] : NINF;
                    float cm = fmaxf(fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[0][2], s[0][3])),
                                     fmaxf(fmaxf(s[1][0], s[1][1]), fmaxf(s[1][2], s[1][3])));
                    cm = redux_max_f32(cm, 0xffffffffu);
                    const float cm2 = cm * kLog2e;
                    float e[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if constexpr (X3) e[c] = __expf(s[0][c] - cm) + (NR == 2 ? __expf(s[1][c] - cm) : 0.f);
                        else e[c] = ex2_approx(fmaf(s[0][c], kLog2e, -cm2)) + (NR == 2 ? ex2_approx(fmaf(s[1][c], kLog2e, -cm2)) : 0.f);
                        e[c] += __shfl_xor_sync(0xffffffffu, e[c], 4);
                        e[c] += __shfl_xor_sync(0xffffffffu, e[c], 8);
                        e[c] += __shfl_xor_sync(0xffffffffu, e[c], 16);
                    }
                    if (g == 0) {
                        imp[jb + 2 * r] = e[0]; imp[jb + 2 * r + 1] = e[1];
                        if (CR > 8) { imp[jb + 8 + 2 * r] = e[2]; imp[jb + 9 + 2 * r] = e[3]; }
                    }
                    if (lane == 0) cmax[a] = cm;
                }
                __syncwarp();
                // common reference maximum (src/naive.py:204-205), right-most candidate forced (src/naive.py:93)
                float M = -INFINITY;
                for (int a = lane; a < np; a += 32) M = fmaxf(M, cmax[a]);
                M = warp_max(M);
                for (int j = lane; j < nc; j += 32) {
                    float v = imp[j] * __expf(cmax[j / CR] - M);
                    if (j == rp) v = kForcedImportance;
                    imp[j] = v;
                }
                __syncwarp();
                // ---- exact Top-K: bitwise search for the TK-th largest key (keys are non-negative floats) ----
                const uint32_t* key = reinterpret_cast<const uint32_t*>(imp);
                uint32_t tau = 0;
                int c_gt = 0;
                if (maxc <= 1024) {
                    // at most 32 keys per lane: they stay in registers for the whole search (padding 0 is below every threshold)
                    uint32_t kreg[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) { const int j = lane + 32 * i; kreg[i] = j < nc ? key[j] : 0u; }
                    for (int bit = 30; bit >= 0; --bit) {
                        const uint32_t cand = tau | (1u << bit);
                        int c = 0;
#pragma unroll
                        for (int i = 0; i < 32; ++i) c += kreg[i] >= cand;
                        c = __reduce_add_sync(0xffffffffu, c);
                        if (c >= TK) tau = cand;
                        if (c == TK) break;   // exactly TK keys reach this threshold: the kept set is decided, lower bits cannot change it
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) c_gt += kreg[i] > tau;
                } else {
                    for (int bit = 30; bit >= 0; --bit) {
                        const uint32_t cand = tau | (1u << bit);
                        int c = 0;
                        for (int j = lane; j < nc; j += 32) c += key[j] >= cand;
                        c = __reduce_add_sync(0xffffffffu, c);
                        if (c >= TK) tau = cand;
                        if (c == TK) break;
                    }
                    for (int j = lane; j < nc; j += 32) c_gt += key[j] > tau;
                }
                c_gt = __reduce_add_sync(0xffffffffu, c_gt);
                const int need = TK - c_gt;     // keys equal to tau that are kept: the smallest positions
                int base_eq = 0, base_out = 0;
                for (int j0 = 0; j0 < nc; j0 += 32) {
                    const int j = j0 + lane;
                    const uint32_t kx = j < nc ? key[j] : 0u;
                    const bool gt = j < nc && kx > tau, eq = j < nc && kx == tau;
                    const uint32_t meq = __ballot_sync(0xffffffffu, eq);
                    const int eq_rank = base_eq + __popc(meq & ((1u << lane) - 1u));
                    const bool keep = gt || (eq && eq_rank < need);
                    const uint32_t mk = __ballot_sync(0xffffffffu, keep);
                    if (keep) nxt[base_out + __popc(mk & ((1u << lane) - 1u))] = par[j / CR] * CR + j % CR;
                    if (lane == 0) selw[j0 >> 5] = mk;
                    base_eq += __popc(meq); base_out += __popc(mk);
                }
                for (int i = base_out + lane; i < TK; i += 32) nxt[i] = -1;
                __syncwarp();
                // ---- pass 2: accumulate what was not kept ----
                if (!select_only) {
                    for (int a = 0; a < np; ++a) {
                        const uint32_t kept = (selw[(a * CR) >> 5] >> ((a * CR) & 31)) & kAllChildren;
                        const uint32_t valid = a == np - 1 ? ((2u << rc) - 1u) : kAllChildren;
                        const uint32_t mask = ~kept & valid;
                        if (mask == 0) continue;
                        float S0[4], S1[4];
                        score(a, S0, S1, false);
                        accumulate_chunk(a, S0, S1, mask);
                    }
                }
            }
            __syncwarp();
            int32_t* tmp = par; par = nxt; nxt = tmp;
        } else {
            if constexpr (PIPE) pipe_begin(np);
            for (int a = 0; a < np; ++a) {
                if constexpr (PIPE) { slot = pipe_next(a, np); if (!slot) return; }
                const uint32_t valid = a == np - 1 ? ((2u << rc) - 1u) : kAllChildren;
                float S0[4], S1[4];
                score(a, S0, S1, false);
                accumulate_chunk(a, S0, S1, valid);
            }
        }
    }
    if (select_only) return;

    // ---- epilogue: out = O / sum in the storage type; (gmax, gsum) for the backward ----
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        s_run[rr] += __shfl_xor_sync(0xffffffffu, s_run[rr], 1);
        s_run[rr] += __shfl_xor_sync(0xffffffffu, s_run[rr], 2);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!row_ok[rr]) continue;
        const float inv = 1.f / s_run[rr];
        if constexpr (X3) {
            // columns 2*VB*r + [0, VB) (element 2rr of the tiles) and the VB after them (element 2rr+1), as fp32
            float* orow = reinterpret_cast<float*>(p.out) + (hbase + g + 8 * rr) * D + 2 * VB * r;
#pragma unroll
            for (int i = 0; i < VB / 4; ++i) {
                reinterpret_cast<float4*>(orow)[i] = make_float4(O[4 * i][2 * rr] * inv, O[4 * i + 1][2 * rr] * inv, O[4 * i + 2][2 * rr] * inv, O[4 * i + 3][2 * rr] * inv);
                reinterpret_cast<float4*>(orow + VB)[i] = make_float4(O[4 * i][2 * rr + 1] * inv, O[4 * i + 1][2 * rr + 1] * inv, O[4 * i + 2][2 * rr + 1] * inv, O[4 * i + 3][2 * rr + 1] * inv);
            }
            if (r == 0) { p.gmax[hbase + g + 8 * rr] = m_true[rr]; p.gsum[hbase + g + 8 * rr] = s_run[rr] * __expf(m_run[rr] - m_true[rr]); }
            continue;
        }
        T* orow = reinterpret_cast<T*>(p.out) + (hbase + g + 8 * rr) * D;
        // this thread owns columns 2*VB*r + [0, VB) (element 2rr of tiles 0..VB-1) and the VB after them (element 2rr+1)
        uint32_t wlo[VB / 2], whi[VB / 2];
#pragma unroll
        for (int i = 0; i < VB / 2; ++i) {
            wlo[i] = F::pack(O[2 * i][2 * rr] * inv, O[2 * i + 1][2 * rr] * inv);
            whi[i] = F::pack(O[2 * i][2 * rr + 1] * inv, O[2 * i + 1][2 * rr + 1] * inv);
        }
        uint4* dst = reinterpret_cast<uint4*>(orow + 2 * VB * r);
#pragma unroll
        for (int i = 0; i < VB / 8; ++i) {
            dst[i] = make_uint4(wlo[4 * i], wlo[4 * i + 1], wlo[4 * i + 2], wlo[4 * i + 3]);
            dst[VB / 8 + i] = make_uint4(whi[4 * i], whi[4 * i + 1], whi[4 * i + 2], whi[4 * i + 3]);
        }
        if (r == 0) { p.gmax[hbase + g + 8 * rr] = m_true[rr]; p.gsum[hbase + g + 8 * rr] = s_run[rr] * __expf(m_run[rr] - m_true[rr]); }
    }
}

template <typename T, int D, bool ROT16, int MODE, int NR, int CR>
static int launch_mma_mode_cr(const AttnParams& p, cudaStream_t st) {
    // pipelined variant where the shape has one and the caller provided the blocked keys
    constexpr bool kHasPipe = D == 128 && CR == 16 && !std::is_same<T, float>::value &&
                              ((MODE == 1 && HTREE_PIPE_SEL) || (MODE == 2 && HTREE_PIPE_ACC));
    if constexpr (kHasPipe) {
        bool pipe = !(p.flags & HTREE_FWD_NO_PIPELINE);
        for (int l = 0; l < p.L; ++l) pipe = pipe && p.lkb[l] != nullptr && (MODE == 1 || p.lvb[l] != nullptr);
        constexpr int W = fwd_warps_per_block(MODE, true, NR);
        const size_t psmem = mma_smem_per_warp(p.TK, CR, MODE != 2, pipe_bytes_per_warp(MODE, ROT16)) * W;
        // the ring must leave room for the intended number of resident blocks (1 KB per block is reserved by the system)
        if (pipe && (psmem + 1024) * fwd_blocks_per_sm(MODE, true, false) <= 227 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(fwd_mma_kernel<T, D, ROT16, MODE, NR, CR, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
            if (e != cudaSuccess) return (int)e;
            dim3 grid((p.Tq + W - 1) / W, p.B * p.Hkv);
            fwd_mma_kernel<T, D, ROT16, MODE, NR, CR, true><<<grid, W * 32, psmem, st>>>(p);
            note_launch();
            return (int)cudaGetLastError();
        }
    }
    constexpr int W0 = fwd_warps_per_block(MODE, false);
    const size_t smem = mma_smem_per_warp(p.TK, CR, MODE != 2) * W0;
    if (smem > 200 * 1024) return HTREE_E_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(fwd_mma_kernel<T, D, ROT16, MODE, NR, CR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((p.Tq + W0 - 1) / W0, p.B * p.Hkv);
    fwd_mma_kernel<T, D, ROT16, MODE, NR, CR><<<grid, W0 * 32, smem, st>>>(p);
    note_launch();
    return (int)cudaGetLastError();
}

template <typename T, int D, bool ROT16, int MODE, int NR>
static int launch_mma_mode_nr(const AttnParams& p, cudaStream_t st) {
    return p.CR == 8 ? launch_mma_mode_cr<T, D, ROT16, MODE, NR, 8>(p, st) : launch_mma_mode_cr<T, D, ROT16, MODE, NR, 16>(p, st);
}

template <typename T, int D, bool ROT16, int MODE>
static int launch_mma_mode(const AttnParams& p, cudaStream_t st) {
    return p.G <= 8 ? launch_mma_mode_nr<T, D, ROT16, MODE, 1>(p, st) : launch_mma_mode_nr<T, D, ROT16, MODE, 2>(p, st);
}

template <typename T, int D, bool ROT16>
static int launch_mma_tdr(const AttnParams& p, cudaStream_t st) {
    if (p.flags & HTREE_FWD_SELECT_ONLY) return launch_mma_mode<T, D, ROT16, 1>(p, st);
    bool have_parents = !(p.flags & HTREE_FWD_FUSED);
    for (int l = 0; l < p.L; ++l) have_parents = have_parents && p.parents[l] != nullptr;
    if (!have_parents) return launch_mma_mode<T, D, ROT16, 0>(p, st);
    const int rc = launch_mma_mode<T, D, ROT16, 1>(p, st);          // selections -> parents[l]
    return rc ? rc : launch_mma_mode<T, D, ROT16, 2>(p, st);         // accumulation given the selections
}

template <typename T, int D>
static int launch_mma_td(const AttnParams& p, cudaStream_t st) {
    return (p.cosh != nullptr && p.sinh != nullptr) ? launch_mma_tdr<T, D, true>(p, st) : launch_mma_tdr<T, D, false>(p, st);
}

bool fwd_mma_supported(const AttnParams& p, int dtype) {
    if (dtype != HTREE_BF16 && dtype != HTREE_F16 && dtype != HTREE_F32) return false;
    if (p.K != p.V || (p.K != 64 && p.K != 128)) return false;
    if (dtype == HTREE_F32 && p.K != 64) return false;     // split-half kernels: 64-wide heads
    if (p.G > 16 || (p.CR != 16 && p.CR != 8)) return false;
    for (int l = 0; l < p.L; ++l) if (!p.lkr[l]) return false;
    if (!(p.flags & HTREE_FWD_SELECT_ONLY))
        for (int l = 0; l < p.L; ++l) if (!p.lvb[l]) return false;
    return mma_smem_per_warp(p.TK, p.CR) * MW <= 200 * 1024;
}

int launch_fwd_mma(const AttnParams& p, int dtype, cudaStream_t st) {
    if (dtype == HTREE_F32) return launch_mma_tdr<float, 64, false>(p, st);
    if (dtype == HTREE_BF16) return p.K == 128 ? launch_mma_td<__nv_bfloat16, 128>(p, st) : launch_mma_td<__nv_bfloat16, 64>(p, st);
    return p.K == 128 ? launch_mma_td<__half, 128>(p, st) : launch_mma_td<__half, 64>(p, st);
}

}  // namespace htree
