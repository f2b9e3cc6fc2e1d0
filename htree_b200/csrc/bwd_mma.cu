// Tensor-core backward for 16-bit storage types, head_dim 128: one WARP per (batch, query position, KV head) group,
// all tree levels in one launch, operands gathered global/L2 -> registers -> mma.sync.
//
// Replaces htree_bwd_preprocess_delta_kernel, htree_bwd_dq_bottom/upper_kernel, htree_bwd_build_parent_mask_kernel and
// htree_bwd_dkv_bottom/upper_kernel (src/backward.py:45-780) for bf16/fp16, K == V in {64, 128}, group <= 16,
// compression_rate 16 or 8.  Arithmetic follows src/naive.py:376-386 with the forward's decomposition
// S = (scale R(p-16a) q)^T K',  K' = R(node % 16) K  (see fwd_mma.cu).  For every accumulated chunk (the 16 children
// of one parent, minus the children the next level kept):
//   S   = q^_a K'^T                                    (score product, as in the forward)
//   P   = exp(S - gmax) / gsum,  dP = dO V^T,  dS = P * (dP - D),  D = sum_v dO * out
//   dq += scale * dS (R(16a-p) K')                     keys re-gathered row-wise, rotated back into q's frame
//   dK'[node] += dS^T q^_a                             one k16 product per 8 columns; fragments transposed with movmatrix
//   dV[node]  += P^T dO
// dK'/dV go to the fp32 level buffers with 16-byte vector reductions (red.global.add.v4.f32) in a layout that lets a
// quad fill whole 32-byte sectors; finalize_grads_kernel afterwards restores the column order and applies
// dK = R(node % 16)^T dK' once per node.  dq stays in registers across all levels and is written once.
#include "mma_common.cuh"

namespace htree {

#ifdef HTREE_BWD_MAXNREG
#define HTREE_BWD_BOUNDS __maxnreg__(HTREE_BWD_MAXNREG)
#else
#define HTREE_BWD_BOUNDS __launch_bounds__(HTREE_BWD_WARPS * 32, HTREE_BWD_MIN_BLOCKS)
#endif
#ifndef HTREE_BWD_WARPS
#define HTREE_BWD_WARPS 4
#endif
constexpr int MWB = HTREE_BWD_WARPS;   // warps (= queries) per block
#ifndef HTREE_BWD_MIN_BLOCKS
#define HTREE_BWD_MIN_BLOCKS 2   // register budget: 2 blocks of 128 threads per SM (255 registers)
#endif

__host__ __device__ inline size_t bwd_mma_smem_per_warp(int TK) { return sizeof(int32_t) * 3 * (size_t)TK; }

// T = float: split-half products (every operand carried as hi + lo half pairs, three MMAs per product; mma_common.cuh),
// 64-wide heads; the K' levels then hold a hi and a lo plane, value rows are read as fp32 and split in registers.
template <typename T, int D, bool ROT16, int NR, int CR>
__global__ void HTREE_BWD_BOUNDS bwd_mma_kernel(const __grid_constant__ AttnParams p) {
    constexpr bool X3 = std::is_same<T, float>::value;
    constexpr bool T1 = CR > 8;   // CR = children per parent: 16, or 8 (then tile 1 stays empty)
    constexpr int HALF = D / 2, KS = D / 16, PPT = HALF / 4, NV = PPT / 8, NOT = D / 8;
    using F = Frag<typename std::conditional<X3, __half, T>::type>;
    using FS = Frag<__half>;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, r = lane & 3;
    const int tl = blockIdx.x * MWB + warp;
    if (tl >= p.Tq) return;                         // warps are independent (no block barrier anywhere)
    const int t = p.t0 + tl;                        // query window: row tl of q / dO / out / dq is sequence position t0 + tl
    const int b = blockIdx.y / p.Hkv, hk = blockIdx.y % p.Hkv;
    const int G = p.G, TK = p.TK, L = p.L;
    int32_t* par = reinterpret_cast<int32_t*>(smem_raw + (size_t)warp * bwd_mma_smem_per_warp(TK));
    int32_t* nsel = par + TK;
    uint32_t* keptw = reinterpret_cast<uint32_t*>(nsel + TK);

    const int64_t hbase = ((int64_t)b * p.Tq + tl) * p.H + (int64_t)hk * G;
    const int64_t qidx = ((int64_t)b * p.Tq + tl) * p.Hkv + hk;
    const bool row_ok[2] = {g < G, NR == 2 && g + 8 < G};   // NR = 1: at most 8 heads, rows g+8 are padding

    // 16-bit types: qraw = IEEE half pairs, dOraw = storage-type pairs.  fp32: qraw = the float bits of q; dOraw / dOlo =
    // the hi and lo half pairs of dO.
    uint32_t qraw[2][2][X3 ? 2 * KS : KS], dOraw[2][2][KS], dOlo[2][2][X3 ? KS : 1];
    constexpr bool rot16 = ROT16;   // packed-half rotations (needs the pre-scaled half tables)
    float Drow[2], gmx[2], ginv[2];
    if constexpr (X3) {
        load_rows_f32<D>(reinterpret_cast<const float*>(p.q) + hbase * D, g, r, row_ok, qraw);
        uint32_t dOf[2][2][2 * KS], of[2][2][2 * KS];
        load_rows_f32<D>(reinterpret_cast<const float*>(p.dO) + hbase * D, g, r, row_ok, dOf);
        load_rows_f32<D>(reinterpret_cast<const float*>(p.out) + hbase * D, g, r, row_ok, of);
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float sdo = 0.f;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const float a0 = __uint_as_float(dOf[rr][hf][2 * ks]), a1 = __uint_as_float(dOf[rr][hf][2 * ks + 1]);
                    sdo += a0 * __uint_as_float(of[rr][hf][2 * ks]) + a1 * __uint_as_float(of[rr][hf][2 * ks + 1]);
                    split_half2(a0, a1, dOraw[rr][hf][ks], dOlo[rr][hf][ks]);
                }
            sdo += __shfl_xor_sync(0xffffffffu, sdo, 1);
            sdo += __shfl_xor_sync(0xffffffffu, sdo, 2);
            Drow[rr] = sdo;
            gmx[rr] = row_ok[rr] ? p.gmax[hbase + g + 8 * rr] : 0.f;
            ginv[rr] = row_ok[rr] ? 1.f / p.gsum[hbase + g + 8 * rr] : 0.f;
        }
    } else {
        load_rows_half<T, D>(reinterpret_cast<const T*>(p.q) + hbase * D, g, r, row_ok, qraw);
        load_rows<T, D>(reinterpret_cast<const T*>(p.dO) + hbase * D, g, r, row_ok, dOraw);
        // D = sum_v dO * out over the whole row (src/naive.py:333); this thread holds 32 of the 128 columns
        uint32_t oraw[2][2][KS];
        load_rows<T, D>(reinterpret_cast<const T*>(p.out) + hbase * D, g, r, row_ok, oraw);
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float sdo = 0.f;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const float2 a = F::unpack(dOraw[rr][hf][ks]), o = F::unpack(oraw[rr][hf][ks]);
                    sdo += a.x * o.x + a.y * o.y;
                }
            sdo += __shfl_xor_sync(0xffffffffu, sdo, 1);
            sdo += __shfl_xor_sync(0xffffffffu, sdo, 2);
            Drow[rr] = sdo;
            gmx[rr] = row_ok[rr] ? p.gmax[hbase + g + 8 * rr] : 0.f;
            ginv[rr] = row_ok[rr] ? 1.f / p.gsum[hbase + g + 8 * rr] : 0.f;
        }
    }

    float dqa[NOT][4];   // dq of rows g, g+8; tile 2*ks + half, columns 2r, 2r+1 <-> dims half*HALF + PPT*r + 2*ks + {0,1}
#pragma unroll
    for (int i = 0; i < NOT; ++i) { dqa[i][0] = dqa[i][1] = dqa[i][2] = dqa[i][3] = 0.f; }

    for (int l = L - 1; l >= 0; --l) {
#ifdef HTREE_BWD_SKIP_LEVEL   // timing experiments only: leaves out one level's work (results are then incomplete)
        if (l == HTREE_BWD_SKIP_LEVEL) continue;
#endif
        const int Nl = p.ln[l];
        const __half* lkr = reinterpret_cast<const __half*>(p.lkr[l]);
        const T* lv = reinterpret_cast<const T*>(p.lv[l]);
        float* dkl = p.dk[l];
        float* dvl = p.dv[l];
        // per-lane bases into this level: only node * rstride is left to add per chunk
        const int rstride = p.Hkv * D;
        constexpr bool stream_rows = true;   // gathered rows are used once: not allocated in L1
        const __half* kq = lkr + ((int64_t)b * Nl * p.Hkv + hk) * D + (D == 64 ? D / 4 : D / 8) * r;
        const T* vq = lv + ((int64_t)b * Nl * p.Hkv + hk) * D + (D / 8) * r;
        const int64_t gbase = ((int64_t)b * Nl * p.Hkv + hk) * D + ((g & 1) ? 16 : 0) + 4 * r;
        __syncwarp();
        for (int i = lane; i < TK; i += 32) {
            par[i] = load_parent(p, l, qidx * TK + i);
            nsel[i] = l > 0 ? load_parent(p, l - 1, qidx * TK + i) : -1;
            keptw[i] = 0u;
        }
        __syncwarp();
        int np = 0;
        for (int i = lane; i < TK; i += 32) np += par[i] >= 0;
        np = __reduce_add_sync(0xffffffffu, np);
        if (np <= 0) continue;
        // children the next level kept: bit c of keptw[a] for node = par[a]*16 + c (both lists ascending)
        for (int i = lane; i < TK; i += 32) {
            const int node = nsel[i];
            if (node < 0) continue;
            const int parent = node / CR;
            int lo = 0, hi = np;
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (par[mid] < parent) lo = mid + 1; else hi = mid; }
            if (lo < np && par[lo] == parent) atomicOr(&keptw[lo], 1u << (node % CR));
        }
        __syncwarp();
        const int rc = (int)(((int64_t)t / p.lpow[l]) % CR);
        const int rp = (np - 1) * CR + rc;

        for (int a = 0; a < np; ++a) {
            const uint32_t valid = a == np - 1 ? ((2u << rc) - 1u) : ((1u << CR) - 1u);
            const uint32_t mask = ~keptw[a] & valid;
            if (mask == 0) continue;
            int node0 = par[a] * CR;
            if (node0 < 0 || node0 >= Nl) { if (p.status) atomicOr(p.status, 8); node0 = 0; }
            const int delta = rp - CR * a;
            const int col[4] = {2 * r, 2 * r + 1, 8 + 2 * r, 9 + 2 * r};
            const bool cv[4] = {(mask >> col[0] & 1) != 0, (mask >> col[1] & 1) != 0, (mask >> col[2] & 1) != 0, (mask >> col[3] & 1) != 0};

            // ---- dP = dO V^T: value rows in the same (column n = child, permuted contraction) fragment order ----
            float dP0[4] = {0.f, 0.f, 0.f, 0.f}, dP1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                // rows beyond the end of the level are read from the last row: their columns are masked below
                const int n0 = min(node0 + g, Nl - 1), n1 = min(node0 + 8 + g, Nl - 1);
                const T* v0 = vq + (int64_t)n0 * rstride;
                const T* v1 = vq + (int64_t)n1 * rstride;
                if constexpr (X3) {
                    // fp32 rows: 8 floats of each half per lane, split into hi / lo half pairs in registers
#pragma unroll
                    for (int tl = 0; tl < (T1 ? 2 : 1); ++tl) {
                        const T* vr = tl ? v1 : v0;
                        uint32_t vf[2][8];
                        ldg_vec<2>(vr, true, vf[0], stream_rows);
                        ldg_vec<2>(vr + HALF, true, vf[1], stream_rows);
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            uint32_t bh[2], bl[2];
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                const float x0 = fminf(fmaxf(__uint_as_float(vf[hf][2 * ks]), -65504.f), 65504.f);
                                const float x1 = fminf(fmaxf(__uint_as_float(vf[hf][2 * ks + 1]), -65504.f), 65504.f);
                                split_half2(x0, x1, bh[hf], bl[hf]);
                            }
                            float (&dP)[4] = tl ? dP1 : dP0;
                            F::mma(dP, dOraw[0][0][ks], dOraw[1][0][ks], dOraw[0][1][ks], dOraw[1][1][ks], bh[0], bh[1]);
                            F::mma(dP, dOraw[0][0][ks], dOraw[1][0][ks], dOraw[0][1][ks], dOraw[1][1][ks], bl[0], bl[1]);
                            F::mma(dP, dOlo[0][0][ks], dOlo[1][0][ks], dOlo[0][1][ks], dOlo[1][1][ks], bh[0], bh[1]);
                        }
                    }
                } else {
                    uint32_t vb[2][2][KS];
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        ldg_vec<NV>(v0 + hf * HALF, true, vb[0][hf], stream_rows);
                        if (T1) ldg_vec<NV>(v1 + hf * HALF, true, vb[1][hf], stream_rows);
                    }
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        F::mma(dP0, dOraw[0][0][ks], dOraw[1][0][ks], dOraw[0][1][ks], dOraw[1][1][ks], vb[0][0][ks], vb[0][1][ks]);
                        if (T1) F::mma(dP1, dOraw[0][0][ks], dOraw[1][0][ks], dOraw[0][1][ks], dOraw[1][1][ks], vb[1][0][ks], vb[1][1][ks]);
                    }
                }
            }

            // ---- S, the rotated-query fragments and the keys rotated back into q's frame ----
            float S0[4], S1[4];
            uint32_t qa[KS][4], qal[X3 ? KS : 1][4];      // rotated-query A fragments (fp32: hi and lo)
            uint32_t kr[2][2][X3 ? 1 : KS];                // 16-bit: keys rotated back, packed half pairs
            float krf[2][2][X3 ? 2 * KS : 1];              // fp32: the same as floats
            if constexpr (X3) score_chunk_x3<D, NR, CR, true>(p, kq, (int64_t)p.B * Nl * rstride, rstride, Nl, node0, delta, g, r, qraw, S0, S1,
                                                             stream_rows, qa, qal, krf);
            else score_chunk<D, true, ROT16, true, NR, CR>(p, kq, rstride, Nl, node0, delta, g, r, qraw, S0, S1, qa, kr, stream_rows);

            // ---- P and dS (src/naive.py:379-382), zero outside the accumulated set ----
            float P[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, dS[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                const float s[2][4] = {{S0[0], S0[1], S1[0], S1[1]}, {S0[2], S0[3], S1[2], S1[3]}};
                const float dp[2][4] = {{dP0[0], dP0[1], dP1[0], dP1[1]}, {dP0[2], dP0[3], dP1[2], dP1[3]}};
#pragma unroll
                for (int rr = 0; rr < NR; ++rr)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const bool on = cv[c] && row_ok[rr];
                        P[rr][c] = on ? __expf(s[rr][c] - gmx[rr]) * ginv[rr] : 0.f;
                        dS[rr][c] = on ? P[rr][c] * (dp[rr][c] - Drow[rr]) : 0.f;
                    }
            }
            // A fragments of dS (heads x children) and, transposed with movmatrix, of dS^T and P^T (children x heads);
            // fp32 storage: hi parts in ds/dst/pt, lo parts in dsl/dstl/ptl
            uint32_t ds[4], dsl[4] = {0u, 0u, 0u, 0u}, pp[4], ppl[4] = {0u, 0u, 0u, 0u};
            if constexpr (X3) {
                split_half2(dS[0][0], dS[0][1], ds[0], dsl[0]); split_half2(dS[1][0], dS[1][1], ds[1], dsl[1]);
                split_half2(dS[0][2], dS[0][3], ds[2], dsl[2]); split_half2(dS[1][2], dS[1][3], ds[3], dsl[3]);
                split_half2(P[0][0], P[0][1], pp[0], ppl[0]); split_half2(P[1][0], P[1][1], pp[1], ppl[1]);
                split_half2(P[0][2], P[0][3], pp[2], ppl[2]); split_half2(P[1][2], P[1][3], pp[3], ppl[3]);
            } else {
                ds[0] = FS::pack(dS[0][0], dS[0][1]); ds[1] = FS::pack(dS[1][0], dS[1][1]);
                ds[2] = FS::pack(dS[0][2], dS[0][3]); ds[3] = FS::pack(dS[1][2], dS[1][3]);
                pp[0] = F::pack(P[0][0], P[0][1]); pp[1] = F::pack(P[1][0], P[1][1]);
                pp[2] = F::pack(P[0][2], P[0][3]); pp[3] = F::pack(P[1][2], P[1][3]);
            }
            const uint32_t ds0 = ds[0], ds1 = ds[1], ds2 = ds[2], ds3 = ds[3];
            const uint32_t dst0 = movmatrix_trans(ds[0]), dst1 = movmatrix_trans(ds[2]);
            const uint32_t dst2 = movmatrix_trans(ds[1]), dst3 = movmatrix_trans(ds[3]);
            const uint32_t pt0 = movmatrix_trans(pp[0]), pt1 = movmatrix_trans(pp[2]);
            const uint32_t pt2 = movmatrix_trans(pp[1]), pt3 = movmatrix_trans(pp[3]);
            uint32_t dstl[4] = {0u, 0u, 0u, 0u}, ptl[4] = {0u, 0u, 0u, 0u};
            if constexpr (X3) {
                dstl[0] = movmatrix_trans(dsl[0]); dstl[1] = movmatrix_trans(dsl[2]); dstl[2] = movmatrix_trans(dsl[1]); dstl[3] = movmatrix_trans(dsl[3]);
                ptl[0] = movmatrix_trans(ppl[0]); ptl[1] = movmatrix_trans(ppl[2]); ptl[2] = movmatrix_trans(ppl[1]); ptl[3] = movmatrix_trans(ppl[3]);
            }

            // ---- dq += dS K~: B fragments = the rotated keys of the score product, transposed in registers ----
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                if constexpr (X3) {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        uint32_t k0h, k0l, k1h, k1l;
                        split_half2(krf[0][hf][2 * ks], krf[0][hf][2 * ks + 1], k0h, k0l);
                        split_half2(krf[1][hf][2 * ks], krf[1][hf][2 * ks + 1], k1h, k1l);
                        const uint32_t b0h = movmatrix_trans(k0h), b1h = movmatrix_trans(k1h);
                        const uint32_t b0l = movmatrix_trans(k0l), b1l = movmatrix_trans(k1l);
                        // summed from zero, then added with a round-to-nearest fp32 add (the tensor core's accumulation
                        // truncates; dq runs over every chunk of the query)
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
                        FS::mma(acc, dsl[0], dsl[1], dsl[2], dsl[3], b0h, b1h);
                        FS::mma(acc, ds0, ds1, ds2, ds3, b0l, b1l);
                        FS::mma(acc, ds0, ds1, ds2, ds3, b0h, b1h);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dqa[2 * ks + hf][i] += acc[i];
                    }
                } else {
                    FS::mma(dqa[2 * ks], ds0, ds1, ds2, ds3, movmatrix_trans(kr[0][0][ks]), movmatrix_trans(kr[1][0][ks]));
                    FS::mma(dqa[2 * ks + 1], ds0, ds1, ds2, ds3, movmatrix_trans(kr[0][1][ks]), movmatrix_trans(kr[1][1][ks]));
                }
            }

            // ---- dK'[node0 + c] += dS^T q^_a and dV[node0 + c] += P^T dO, rows c = g and g + 8 ----
            // The level buffers are used in a private layout here: dK' is the gradient of the pre-rotated key (the
            // rotation by the child index is undone once per node by finalize_grads_kernel, not once per visit), and
            // position 32*m + 16*half + 4*r + i of a row holds column half*D/2 + (D/8)*r + 4*m + i.
            // Rows are written by PAIRS of quads: lanes of rows g and g^1 swap one half each, so that the 8 lanes write
            // 128 contiguous bytes (a whole cache line) of ONE row per instruction: position 32*m + 16*half + 4*r + i.
            const bool odd = (g & 1) != 0;
            const int ge = g & ~1;
            bool rowa[2], rowb[2];
            float* dka[2]; float* dkb[2]; float* dva[2]; float* dvb[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                rowa[rr] = (mask >> (ge + 8 * rr) & 1) != 0;          // even row of the pair
                rowb[rr] = (mask >> (ge + 1 + 8 * rr) & 1) != 0;      // odd row of the pair
                const int64_t offa = gbase + (int64_t)(node0 + ge + 8 * rr) * rstride;
                const int64_t offb = offa + rstride;
                dka[rr] = dkl + offa; dkb[rr] = dkl + offb;
                dva[rr] = dvl + offa; dvb[rr] = dvl + offb;
            }
#pragma unroll
            for (int m = 0; m < KS / 2; ++m) {
                float klo_[2][4], khi_[2][4], vlo_[2][4], vhi_[2][4];   // [row][4 consecutive columns 16r + 4m + i]
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int ks = 2 * m + u;
                    float tl_[4] = {0.f, 0.f, 0.f, 0.f}, th_[4] = {0.f, 0.f, 0.f, 0.f};
                    float ul_[4] = {0.f, 0.f, 0.f, 0.f}, uh_[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t q0 = movmatrix_trans(qa[ks][0]), q1 = movmatrix_trans(qa[ks][1]);
                    const uint32_t q2 = movmatrix_trans(qa[ks][2]), q3 = movmatrix_trans(qa[ks][3]);
                    const uint32_t o0 = movmatrix_trans(dOraw[0][0][ks]), o1 = movmatrix_trans(dOraw[1][0][ks]);
                    const uint32_t o2 = movmatrix_trans(dOraw[0][1][ks]), o3 = movmatrix_trans(dOraw[1][1][ks]);
                    FS::mma(tl_, dst0, dst1, dst2, dst3, q0, q1);
                    FS::mma(th_, dst0, dst1, dst2, dst3, q2, q3);
                    F::mma(ul_, pt0, pt1, pt2, pt3, o0, o1);
                    F::mma(uh_, pt0, pt1, pt2, pt3, o2, o3);
                    if constexpr (X3) {
                        const uint32_t ql0 = movmatrix_trans(qal[ks][0]), ql1 = movmatrix_trans(qal[ks][1]);
                        const uint32_t ql2 = movmatrix_trans(qal[ks][2]), ql3 = movmatrix_trans(qal[ks][3]);
                        const uint32_t ol0 = movmatrix_trans(dOlo[0][0][ks]), ol1 = movmatrix_trans(dOlo[1][0][ks]);
                        const uint32_t ol2 = movmatrix_trans(dOlo[0][1][ks]), ol3 = movmatrix_trans(dOlo[1][1][ks]);
                        FS::mma(tl_, dst0, dst1, dst2, dst3, ql0, ql1);
                        FS::mma(tl_, dstl[0], dstl[1], dstl[2], dstl[3], q0, q1);
                        FS::mma(th_, dst0, dst1, dst2, dst3, ql2, ql3);
                        FS::mma(th_, dstl[0], dstl[1], dstl[2], dstl[3], q2, q3);
                        F::mma(ul_, pt0, pt1, pt2, pt3, ol0, ol1);
                        F::mma(ul_, ptl[0], ptl[1], ptl[2], ptl[3], o0, o1);
                        F::mma(uh_, pt0, pt1, pt2, pt3, ol2, ol3);
                        F::mma(uh_, ptl[0], ptl[1], ptl[2], ptl[3], o2, o3);
                    }
                    klo_[0][2 * u] = tl_[0]; klo_[0][2 * u + 1] = tl_[1]; klo_[1][2 * u] = tl_[2]; klo_[1][2 * u + 1] = tl_[3];
                    khi_[0][2 * u] = th_[0]; khi_[0][2 * u + 1] = th_[1]; khi_[1][2 * u] = th_[2]; khi_[1][2 * u + 1] = th_[3];
                    vlo_[0][2 * u] = ul_[0]; vlo_[0][2 * u + 1] = ul_[1]; vlo_[1][2 * u] = ul_[2]; vlo_[1][2 * u + 1] = ul_[3];
                    vhi_[0][2 * u] = uh_[0]; vhi_[0][2 * u + 1] = uh_[1]; vhi_[1][2 * u] = uh_[2]; vhi_[1][2 * u + 1] = uh_[3];
                }
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    float ka[4], kb_[4], va[4], vb_[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // even lanes give away their high half and receive the partner's low half; odd lanes the reverse
                        const float rk = __shfl_xor_sync(0xffffffffu, odd ? klo_[rr][i] : khi_[rr][i], 4);
                        const float rv = __shfl_xor_sync(0xffffffffu, odd ? vlo_[rr][i] : vhi_[rr][i], 4);
                        ka[i] = odd ? rk : klo_[rr][i];  kb_[i] = odd ? khi_[rr][i] : rk;
                        va[i] = odd ? rv : vlo_[rr][i];  vb_[i] = odd ? vhi_[rr][i] : rv;
                    }
                    if (rowa[rr]) {
                        red_add_v4(dka[rr] + 32 * m, ka[0], ka[1], ka[2], ka[3]);
                        red_add_v4(dva[rr] + 32 * m, va[0], va[1], va[2], va[3]);
                    }
                    if (rowb[rr]) {
                        red_add_v4(dkb[rr] + 32 * m, kb_[0], kb_[1], kb_[2], kb_[3]);
                        red_add_v4(dvb[rr] + 32 * m, vb_[0], vb_[1], vb_[2], vb_[3]);
                    }
                }
            }
        }
    }

    // ---- dq: this thread owns columns PPT*r + [0, PPT) of both halves of rows g and g+8 ----
    // fp32 (the reference's contract, src/backward.py:1119), or rounded once to the storage type when the caller asked for
    // typed gradients (the cast of src/backward.py:1193 without an fp32 tensor in between)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!row_ok[rr]) continue;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            if (!X3 && p.dq_typed) {
                T* dqrow = reinterpret_cast<T*>(p.dq_typed) + (hbase + g + 8 * rr) * D + hf * HALF + PPT * r;
                uint32_t w[PPT / 2];
#pragma unroll
                for (int m = 0; m < KS / 2; ++m) {
                    w[2 * m] = F::pack(dqa[2 * (2 * m) + hf][2 * rr], dqa[2 * (2 * m) + hf][2 * rr + 1]);
                    w[2 * m + 1] = F::pack(dqa[2 * (2 * m + 1) + hf][2 * rr], dqa[2 * (2 * m + 1) + hf][2 * rr + 1]);
                }
#pragma unroll
                for (int i = 0; i < PPT / 8; ++i)
                    reinterpret_cast<uint4*>(dqrow)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            } else {
                float* dqf = (X3 && p.dq_typed) ? reinterpret_cast<float*>(p.dq_typed) : p.dq;
                float4* dst = reinterpret_cast<float4*>(dqf + (hbase + g + 8 * rr) * D + hf * HALF + PPT * r);
#pragma unroll
                for (int m = 0; m < KS / 2; ++m)
                    dst[m] = make_float4(dqa[2 * (2 * m) + hf][2 * rr], dqa[2 * (2 * m) + hf][2 * rr + 1],
                                         dqa[2 * (2 * m + 1) + hf][2 * rr], dqa[2 * (2 * m + 1) + hf][2 * rr + 1]);
            }
        }
    }
}

// Turns the private accumulator layout of bwd_mma_kernel into gradients, in place, one 16-lane group per row:
// un-permute both buffers (position 32m + 16*half + 4r + i <-> column half*D/2 + (D/8)*r + 4m + i) and rotate dK' back by the
// node's child index, dK = R(node % CR)^T dK' (inverse of the rotation in rotate_keys_kernel; src/naive.py:31-38).
template <int D>
__global__ void __launch_bounds__(256) finalize_grads_kernel(float* dk, float* dv, const float* cosc, const float* sinc,
                                                             int64_t rows, int Hkv, int N, int CR) {
    constexpr int HALF = D / 2, PPT = HALF / 4, LPR = HALF / 4;   // LPR lanes per row: one float4 of each half per lane
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t row = tid / LPR;
    const int j = (int)(tid % LPR);                      // position group 4j .. 4j+3 of each half
    const bool on = row < rows;
    const int m = j >> 2, r = j & 3;
    const int col = PPT * r + 4 * m;                     // first of the 4 columns stored at positions 4j .. 4j+3
    float4 klo = make_float4(0, 0, 0, 0), khi = klo, vlo = klo, vhi = klo;
    float* dkr = dk + row * D;
    float* dvr = dv + row * D;
    if (on) {
        const int pos = 32 * m + 4 * r;                  // low-half piece; the high-half piece follows 16 floats later
        klo = *reinterpret_cast<const float4*>(dkr + pos); khi = *reinterpret_cast<const float4*>(dkr + pos + 16);
        vlo = *reinterpret_cast<const float4*>(dvr + pos); vhi = *reinterpret_cast<const float4*>(dvr + pos + 16);
    }
    __syncwarp();                                        // every lane of the row has read before anyone writes
    if (!on) return;
    const int c = (int)((row / Hkv) % N) % CR;
    const float4 cs = __ldg(reinterpret_cast<const float4*>(cosc + (size_t)c * HALF + col));
    const float4 sn = __ldg(reinterpret_cast<const float4*>(sinc + (size_t)c * HALF + col));
    float4 lo, hi;
    lo.x = klo.x * cs.x + khi.x * sn.x; hi.x = khi.x * cs.x - klo.x * sn.x;
    lo.y = klo.y * cs.y + khi.y * sn.y; hi.y = khi.y * cs.y - klo.y * sn.y;
    lo.z = klo.z * cs.z + khi.z * sn.z; hi.z = khi.z * cs.z - klo.z * sn.z;
    lo.w = klo.w * cs.w + khi.w * sn.w; hi.w = khi.w * cs.w - klo.w * sn.w;
    *reinterpret_cast<float4*>(dkr + col) = lo; *reinterpret_cast<float4*>(dkr + HALF + col) = hi;
    *reinterpret_cast<float4*>(dvr + col) = vlo; *reinterpret_cast<float4*>(dvr + HALF + col) = vhi;
}

bool bwd_mma_supported(const AttnParams& p, int dtype) {
    if (dtype != HTREE_BF16 && dtype != HTREE_F16 && dtype != HTREE_F32) return false;
    if (p.K != p.V || (p.K != 64 && p.K != 128) || p.G > 16 || (p.CR != 16 && p.CR != 8)) return false;
    if (dtype == HTREE_F32 && p.K != 64) return false;     // split-half kernels: 64-wide heads
    for (int l = 0; l < p.L; ++l) if (!p.lkr[l]) return false;
    return bwd_mma_smem_per_warp(p.TK) * MWB <= 200 * 1024;
}

template <typename T, int D, bool ROT16, int NR, int CR>
static int launch_bwd_mma_cr(const AttnParams& p, cudaStream_t st) {
    const size_t smem = bwd_mma_smem_per_warp(p.TK) * MWB;
    dim3 grid((p.Tq + MWB - 1) / MWB, p.B * p.Hkv);
    cudaError_t e = cudaFuncSetAttribute(bwd_mma_kernel<T, D, ROT16, NR, CR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    bwd_mma_kernel<T, D, ROT16, NR, CR><<<grid, MWB * 32, smem, st>>>(p);
    note_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (p.flags & HTREE_BWD_NO_FOLD) return 0;      // more query windows follow: the accumulators stay in their private layout
    for (int l = 0; l < p.L; ++l) {
        const int64_t rows = (int64_t)p.B * p.ln[l] * p.Hkv;
        const unsigned blocks = (unsigned)((rows * (D / 8) + 255) / 256);
        finalize_grads_kernel<D><<<blocks, 256, 0, st>>>(p.dk[l], p.dv[l], p.cosc, p.sinc, rows, p.Hkv, p.ln[l], p.CR);
        note_launch();
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

template <typename T, int D, bool ROT16, int NR>
static int launch_bwd_mma_nr(const AttnParams& p, cudaStream_t st) {
    return p.CR == 8 ? launch_bwd_mma_cr<T, D, ROT16, NR, 8>(p, st) : launch_bwd_mma_cr<T, D, ROT16, NR, 16>(p, st);
}

template <typename T, int D, bool ROT16>
static int launch_bwd_mma_t(const AttnParams& p, cudaStream_t st) {
    return p.G <= 8 ? launch_bwd_mma_nr<T, D, ROT16, 1>(p, st) : launch_bwd_mma_nr<T, D, ROT16, 2>(p, st);
}

int launch_bwd_mma(const AttnParams& p, int dtype, cudaStream_t st) {
    if (dtype == HTREE_F32) return launch_bwd_mma_t<float, 64, false>(p, st);
    const bool rot16 = p.cosh != nullptr && p.sinh != nullptr;
    if (p.K == 128) {
        if (dtype == HTREE_BF16) return rot16 ? launch_bwd_mma_t<__nv_bfloat16, 128, true>(p, st) : launch_bwd_mma_t<__nv_bfloat16, 128, false>(p, st);
        return rot16 ? launch_bwd_mma_t<__half, 128, true>(p, st) : launch_bwd_mma_t<__half, 128, false>(p, st);
    }
    if (dtype == HTREE_BF16) return rot16 ? launch_bwd_mma_t<__nv_bfloat16, 64, true>(p, st) : launch_bwd_mma_t<__nv_bfloat16, 64, false>(p, st);
    return rot16 ? launch_bwd_mma_t<__half, 64, true>(p, st) : launch_bwd_mma_t<__half, 64, false>(p, st);
}

}  // namespace htree
