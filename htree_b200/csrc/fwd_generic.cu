// Storage-type-generic forward: one thread block per (batch, query position, KV head) walks every tree level from the
// top down in a single launch, with fp32 arithmetic throughout.  It is the path for fp32 inputs and for shapes the
// tensor-core kernel was not built for, and it also produces the per-level trace.
//
// Per level (behaviour of src/naive.py:180-223; the reference's GPU kernels are
// htree_select_accumulate_gqa_kernel / htree_bottom_accumulate_gqa_kernel / htree_merge_to_global_kernel /
// htree_final_normalize_kernel, src/parallel.py:248-867):
//   1. rotate + scale the G query heads for position nc-1, keep them transposed in shared memory;
//   2. one thread per candidate: gather its K row, rotate it by the candidate's position, dot with all heads;
//   3. upper levels: shared importance sum_h exp(S - max), exact Top-K by a bitwise search for the K-th largest
//      key, ties resolved to the smaller position, right-most candidate forced in; the kept nodes (already in
//      ascending order) become the next level's parents;
//   4. every candidate that was not kept is accumulated: p = exp(S - rowmax), out += p * V;
//   5. the level state is merged into the running (max, sum, out) state with the reference's 1e-10 guards.
// After the leaf level out/sum is written in the storage type together with (gmax, gsum).
#include "common.cuh"

namespace htree {

constexpr int NT = 256;   // threads per block

struct FwdSmem {
    float* qT;      // [K][GPAD]   rotated, scaled queries, head-minor
    float* S;       // [maxc][RS]  scores, later probabilities (RS = GPAD + 4: conflict-free 16-byte rows);
                    // tiled variant: [NT][RS], the scores of one tile of candidates
    float* mj;      // [maxc]      tiled variant only: per-candidate score maximum of the selection pass
    uint32_t* key;  // [maxc]      importance bit patterns
    uint8_t* sel;   // [maxc]
    int32_t* par;   // [2][TK]
    float* gout;    // [GPAD][V]
    float* lo;      // [GPAD][V]
    float* part;    // [NT][GP]    per-slice partial outputs
    float* red;     // [NT/32][GPAD]
    float* st;      // gm, gs, lm, ls, sg, sc: 6 x [GPAD]
    int* wtot;      // [NT/32]
    int* cnt;       // [4]
};

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

__host__ __device__ inline size_t fwd_smem_layout(int K, int V, int GPAD, int GP, int maxc, int TK, bool tiled, FwdSmem* m,
                                                  unsigned char* base) {
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t r = o; o = align16(o + bytes); return r; };
    size_t a_qT = take(sizeof(float) * K * GPAD);
    size_t a_S = take(sizeof(float) * (size_t)(tiled ? NT : maxc) * (GPAD + 4));
    size_t a_mj = take(tiled ? sizeof(float) * maxc : 0);
    size_t a_key = take(sizeof(uint32_t) * maxc);
    size_t a_sel = take(maxc);
    size_t a_par = take(sizeof(int32_t) * 2 * TK);
    size_t a_gout = take(sizeof(float) * GPAD * V);
    size_t a_lo = take(sizeof(float) * GPAD * V);
    size_t a_part = take(sizeof(float) * NT * GP);
    size_t a_red = take(sizeof(float) * (NT / 32) * GPAD);
    size_t a_st = take(sizeof(float) * 6 * GPAD);
    size_t a_wtot = take(sizeof(int) * (NT / 32));
    size_t a_cnt = take(sizeof(int) * 4);
    if (m) {
        m->qT = (float*)(base + a_qT); m->S = (float*)(base + a_S); m->mj = (float*)(base + a_mj); m->key = (uint32_t*)(base + a_key);
        m->sel = (uint8_t*)(base + a_sel); m->par = (int32_t*)(base + a_par); m->gout = (float*)(base + a_gout);
        m->lo = (float*)(base + a_lo); m->part = (float*)(base + a_part); m->red = (float*)(base + a_red);
        m->st = (float*)(base + a_st); m->wtot = (int*)(base + a_wtot); m->cnt = (int*)(base + a_cnt);
    }
    return o;
}

// Scores of ONE candidate against GP query heads (head chunk starting at g0): rotate the key row by the candidate's
// position, dot with the rotated queries held head-minor in shared memory (src/naive.py:193-199).
template <typename T, int GP>
__device__ __forceinline__ void score_row(const float* qT, int GPAD, int g0, const T* kr, const float* cj, const float* sj,
                                          int half, float (&acc)[GP]) {
#pragma unroll
    for (int g = 0; g < GP; ++g) acc[g] = 0.f;
    for (int d = 0; d < half; d += 4) {
        float lo[4], hi[4];
        load4<T>(kr + d, lo);
        load4<T>(kr + d + half, hi);
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(cj + d));
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(sj + d));
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float klo = lo[u] * cs[u] - hi[u] * sn[u];
            const float khi = lo[u] * sn[u] + hi[u] * cs[u];
            const float* qa = qT + (d + u) * GPAD + g0;
            const float* qb = qT + (d + u + half) * GPAD + g0;
#pragma unroll
            for (int g = 0; g < GP; g += 4) {
                const float4 x = *reinterpret_cast<const float4*>(qa + g);
                const float4 y = *reinterpret_cast<const float4*>(qb + g);
                acc[g] += x.x * klo; acc[g + 1] += x.y * klo; acc[g + 2] += x.z * klo; acc[g + 3] += x.w * klo;
                acc[g] += y.x * khi; acc[g + 1] += y.y * khi; acc[g + 2] += y.z * khi; acc[g + 3] += y.w * khi;
            }
        }
    }
}

// Block-wide count of keys >= thr among key[0..nc).  `slot` rotates over three shared counters so that one barrier
// per call is enough (the counter used two calls ago is cleared here).
__device__ __forceinline__ int count_ge(const uint32_t* key, int nc, uint32_t thr, int* cnt, int& slot) {
    int c = 0;
    for (int j = threadIdx.x; j < nc; j += NT) c += key[j] >= thr;
    c = __reduce_add_sync(0xffffffffu, c);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(&cnt[slot], c);
    __syncthreads();
    int r = cnt[slot];
    int nxt = slot == 2 ? 0 : slot + 1;
    int prev = slot == 0 ? 2 : slot - 1;
    if (threadIdx.x == 0) cnt[prev] = 0;
    slot = nxt;
    return r;
}

// TILED: the level's scores do not fit into shared memory (large top_k * compression_rate * group).  The selection pass
// then keeps only a (maximum, sum of exponentials) pair per candidate and the accumulation pass re-scores the
// candidates tile by tile with an online softmax, instead of holding every score of the level.
template <typename T, int GP, bool TILED>
__global__ void __launch_bounds__(NT) fwd_generic_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, V = p.V, CR = p.CR, TK = p.TK, G = p.G, L = p.L, half = K >> 1;
    const int GPAD = (G + GP - 1) / GP * GP, RS = GPAD + 4, maxc = TK * CR;
    FwdSmem m;
    fwd_smem_layout(K, V, GPAD, GP, maxc, TK, TILED, &m, smem_raw);
    float *gm = m.st, *gs = m.st + GPAD, *lm = m.st + 2 * GPAD, *ls = m.st + 3 * GPAD, *sg = m.st + 4 * GPAD, *sc = m.st + 5 * GPAD;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = p.t0 + blockIdx.x;                                        // sequence position of this query
    const int b = blockIdx.y / p.Hkv, hk = blockIdx.y % p.Hkv;
    const bool select_only = (p.flags & HTREE_FWD_SELECT_ONLY) != 0;
    const int64_t hbase = ((int64_t)b * p.Tq + blockIdx.x) * p.H + (int64_t)hk * G;   // first head of the group
    const int64_t qidx = ((int64_t)b * p.Tq + blockIdx.x) * p.Hkv + hk;               // group index for parents
    const T* qg = reinterpret_cast<const T*>(p.q) + hbase * K;

    // ---- state initialisation (src/parallel.py:995-997, 1026-1038) ----
    for (int i = tid; i < GPAD; i += NT) { gm[i] = kNegInf; gs[i] = 0.f; }
    for (int i = tid; i < GPAD * V; i += NT) m.gout[i] = 0.f;
    if (tid < 4) m.cnt[tid] = 0;
    int32_t* par = m.par;
    int32_t* nxt = m.par + TK;
    if (p.level_mode) {
        for (int i = tid; i < TK; i += NT) par[i] = p.parents_in[qidx * TK + i];
    } else {
        int np0 = (int)(((int64_t)t / p.lpow[L - 1]) / CR) + 1;
        if (np0 > TK) np0 = TK;
        for (int i = tid; i < TK; i += NT) par[i] = i < np0 ? i : -1;
    }
    int slot = 0;
    __syncthreads();

    const int l_hi = p.level_mode ? p.level_index : L - 1, l_lo = p.level_mode ? p.level_index : 0;
    for (int l = l_hi; l >= l_lo; --l) {
        const int Nl = p.ln[l];
        const int64_t tslot = p.level_mode ? 0 : l;   // slot of this level in the trace arrays
        const T* lk = reinterpret_cast<const T*>(p.lk[l]);
        const T* lv = reinterpret_cast<const T*>(p.lv[l]);
        if (p.parents[l]) for (int i = tid; i < TK; i += NT) store_parent(p, l, qidx * TK + i, par[i]);
        if (select_only && l == 0) break;   // the leaf level selects nothing
        int np = 0;   // parents are a dense prefix followed by -1 padding
        for (int i = tid; i < TK; i += NT) np += par[i] >= 0;
        np = __reduce_add_sync(0xffffffffu, np);
        if (lane == 0) m.wtot[warp] = np;
        __syncthreads();
        np = 0;
#pragma unroll
        for (int i = 0; i < NT / 32; ++i) np += m.wtot[i];
        const int rci = (int)(((int64_t)t / p.lpow[l]) % CR);
        // A parent list without entries (only possible in single-level mode, where the caller supplies the lists) is an
        // empty level: no candidate, no rotation position; the level state comes out neutral and the next list empty.
        const bool empty = np <= 0;
        const int nc = empty ? 0 : (np - 1) * CR + rci + 1, rp = nc - 1;

        // ---- 1. queries: rotate by the right-most position, scale, store head-minor ----
        for (int i = tid; i < GPAD * half; i += NT) {
            const int g = i / half, d = i - g * half;
            float a = 0.f, c = 0.f;
            if (g < G && !empty) {
                const float lo = to_f(qg[(int64_t)g * K + d]), hi = to_f(qg[(int64_t)g * K + d + half]);
                const float cs = __ldg(p.cosc + (int64_t)rp * half + d), sn = __ldg(p.sinc + (int64_t)rp * half + d);
                a = (lo * cs - hi * sn) * p.scale;
                c = (lo * sn + hi * cs) * p.scale;
            }
            m.qT[d * GPAD + g] = a;
            m.qT[(d + half) * GPAD + g] = c;
        }
        __syncthreads();   // also orders the wtot reads above before their next use

        // ---- 2. scores: one candidate per thread ----
        float tmax = -INFINITY;
        const bool need_scores = !TILED || (l > 0 && nc > TK);     // the tiled variant scores the leaves while accumulating
        if (need_scores) {
            for (int j = tid; j < nc; j += NT) {
                int node = par[j / CR] * CR + j % CR;
                if (node < 0 || node >= Nl) { if (p.status) atomicOr(p.status, 1); node = 0; }
                const T* kr = lk + (((int64_t)b * Nl + node) * p.Hkv + hk) * K;
                const float* cj = p.cosc + (int64_t)j * half;
                const float* sj = p.sinc + (int64_t)j * half;
                float mrow = -INFINITY, erow = 0.f;   // tiled: running maximum and sum of exp over the head chunks
                for (int g0 = 0; g0 < GPAD; g0 += GP) {
                    float acc[GP];
                    score_row<T, GP>(m.qT, GPAD, g0, kr, cj, sj, half, acc);
                    if (!TILED) {
#pragma unroll
                        for (int g = 0; g < GP; g += 4)
                            *reinterpret_cast<float4*>(m.S + (size_t)j * RS + g0 + g) = make_float4(acc[g], acc[g + 1], acc[g + 2], acc[g + 3]);
#pragma unroll
                        for (int g = 0; g < GP; ++g) if (g0 + g < G) tmax = fmaxf(tmax, acc[g]);
                    } else {
                        float cmx = -INFINITY;
#pragma unroll
                        for (int g = 0; g < GP; ++g) if (g0 + g < G) cmx = fmaxf(cmx, acc[g]);
                        const float mn = fmaxf(mrow, cmx);
                        float e = erow * expf(mrow - mn);
#pragma unroll
                        for (int g = 0; g < GP; ++g) if (g0 + g < G) e += expf(acc[g] - mn);
                        mrow = mn; erow = e;
                    }
                }
                if (TILED) { m.mj[j] = mrow; m.key[j] = __float_as_uint(erow); tmax = fmaxf(tmax, mrow); }
            }
        }

        bool accumulate = true;   // does this level accumulate anything?
        if (l > 0) {
            // ---- 3. shared importance and exact Top-K ----
            tmax = warp_max(tmax);
            if (lane == 0) m.red[warp] = tmax;
            __syncthreads();
            float M = m.red[0];
#pragma unroll
            for (int i = 1; i < NT / 32; ++i) M = fmaxf(M, m.red[i]);
            if (need_scores) {
                for (int j = tid; j < nc; j += NT) {
                    float s = 0.f;
                    if (!TILED) { for (int g = 0; g < G; ++g) s += expf(m.S[(size_t)j * RS + g] - M); }
                    else s = __uint_as_float(m.key[j]) * expf(m.mj[j] - M);
                    if (j == rp) s = kForcedImportance;
                    m.key[j] = __float_as_uint(s);   // s >= 0, so the bit pattern orders like the value
                }
            }
            __syncthreads();
            if (nc <= TK) {
                accumulate = false;
                for (int j = tid; j < TK; j += NT) nxt[j] = j < nc ? par[j / CR] * CR + j % CR : -1;
                for (int j = tid; j < nc; j += NT) m.sel[j] = 1;
            } else {
                uint32_t tau = 0;   // becomes the TK-th largest key
                for (int bit = 30; bit >= 0; --bit) {
                    const uint32_t cand = tau | (1u << bit);
                    const int c_ge = count_ge(m.key, nc, cand, m.cnt, slot);
                    if (c_ge >= TK) tau = cand;
                    if (c_ge == TK) break;   // the kept set is decided: lower bits cannot change it (uniform across the block)
                }
                const int c_gt = tau == 0xffffffffu ? 0 : count_ge(m.key, nc, tau + 1u, m.cnt, slot);
                const int need = TK - c_gt;   // keys equal to tau that are kept: the `need` smallest positions
                int base_eq = 0, base_out = 0;
                for (int j0 = 0; j0 < nc; j0 += NT) {
                    const int j = j0 + tid;
                    const uint32_t key = j < nc ? m.key[j] : 0u;
                    const bool gt = j < nc && key > tau, eq = j < nc && key == tau;
                    int tot_eq, tot_s;
                    const int eq_rank = base_eq + block_scan_flag<NT>(eq, m.wtot, &tot_eq);
                    const bool s = gt || (eq && eq_rank < need);
                    const int pos = base_out + block_scan_flag<NT>(s, m.wtot, &tot_s);
                    if (j < nc) m.sel[j] = s;
                    if (s) nxt[pos] = par[j / CR] * CR + j % CR;
                    base_eq += tot_eq; base_out += tot_s;
                }
                for (int i = base_out + tid; i < TK; i += NT) nxt[i] = -1;
            }
            __syncthreads();
        } else {
            for (int j = tid; j < nc; j += NT) m.sel[j] = 0;
            __syncthreads();
        }

        if (!select_only) {
            // ---- 4. accumulate the candidates that were not kept ----
            if (TILED && accumulate) {
                float* al = sg;   // per-head rescale factor of the running level state (sg is free until the merge)
                for (int g = tid; g < GPAD; g += NT) { lm[g] = kNegInf; ls[g] = 0.f; }
                for (int i = tid; i < GPAD * V; i += NT) m.lo[i] = 0.f;
                __syncthreads();
                const int vcols = V < NT ? V : NT;
                const int nsl = NT / vcols;
                const int slice = tid / vcols, dcol = tid - slice * vcols;
                for (int j0 = 0; j0 < nc; j0 += NT) {
                    const int j = j0 + tid;
                    const bool act = j < nc && !m.sel[j];
                    // scores of this thread's candidate -> tile row tid (-inf when there is nothing to accumulate)
                    {
                        int node = act ? par[j / CR] * CR + j % CR : 0;
                        if (node < 0 || node >= Nl) { if (p.status) atomicOr(p.status, 1); node = 0; }
                        const T* kr = lk + (((int64_t)b * Nl + node) * p.Hkv + hk) * K;
                        const float* cj = p.cosc + (int64_t)(act ? j : 0) * half;
                        const float* sj = p.sinc + (int64_t)(act ? j : 0) * half;
                        for (int g0 = 0; g0 < GPAD; g0 += GP) {
                            float acc[GP];
                            if (act) score_row<T, GP>(m.qT, GPAD, g0, kr, cj, sj, half, acc);
#pragma unroll
                            for (int g = 0; g < GP; ++g) {
                                const float sv = act ? acc[g] : -INFINITY;
                                m.S[(size_t)tid * RS + g0 + g] = sv;
                                const float w = warp_max(sv);
                                if (lane == 0) m.red[warp * GPAD + g0 + g] = w;
                            }
                        }
                    }
                    __syncthreads();
                    for (int g = tid; g < GPAD; g += NT) {
                        float w = m.red[g];
                        for (int i = 1; i < NT / 32; ++i) w = fmaxf(w, m.red[i * GPAD + g]);
                        const float mn = fmaxf(lm[g], w);
                        al[g] = expf(lm[g] - mn);
                        lm[g] = mn;
                    }
                    __syncthreads();
                    for (int g = 0; g < GPAD; ++g) {   // probabilities in place, tile sums
                        float* sp = m.S + (size_t)tid * RS + g;
                        const float pr = act ? expf(*sp - lm[g]) : 0.f;
                        *sp = pr;
                        const float w = warp_sum(pr);
                        if (lane == 0) m.red[warp * GPAD + g] = w;
                    }
                    __syncthreads();
                    for (int g = tid; g < GPAD; g += NT) {
                        float w = 0.f;
                        for (int i = 0; i < NT / 32; ++i) w += m.red[i * GPAD + g];
                        ls[g] = ls[g] * al[g] + w;
                    }
                    const int rows = min(NT, nc - j0);
                    for (int g0 = 0; g0 < GPAD; g0 += GP) {
                        for (int d0 = 0; d0 < V; d0 += vcols) {
                            const int d = d0 + dcol;
                            float acc[GP];
#pragma unroll
                            for (int g = 0; g < GP; ++g) acc[g] = 0.f;
                            if (slice < nsl && d < V) {
                                for (int u = slice; u < rows; u += nsl) {
                                    const int ju = j0 + u;
                                    if (m.sel[ju]) continue;
                                    int node = par[ju / CR] * CR + ju % CR;
                                    if (node < 0 || node >= Nl) node = 0;
                                    const float vv = to_f(lv[(((int64_t)b * Nl + node) * p.Hkv + hk) * V + d]);
                                    const float* pr = m.S + (size_t)u * RS + g0;
#pragma unroll
                                    for (int g = 0; g < GP; g += 4) {
                                        const float4 x = *reinterpret_cast<const float4*>(pr + g);
                                        acc[g] += x.x * vv; acc[g + 1] += x.y * vv; acc[g + 2] += x.z * vv; acc[g + 3] += x.w * vv;
                                    }
                                }
                            }
#pragma unroll
                            for (int g = 0; g < GP; ++g) m.part[tid * GP + g] = acc[g];
                            __syncthreads();
                            for (int i = tid; i < GP * vcols; i += NT) {
                                const int g = i / vcols, dc = i - g * vcols;
                                if (d0 + dc < V) {
                                    float w = 0.f;
                                    for (int s2 = 0; s2 < nsl; ++s2) w += m.part[(s2 * vcols + dc) * GP + g];
                                    float* o = m.lo + (g0 + g) * V + d0 + dc;
                                    *o = *o * al[g0 + g] + w;
                                }
                            }
                            __syncthreads();
                        }
                    }
                }
            } else if (accumulate) {
                for (int g0 = 0; g0 < GPAD; g0 += GP) {   // row maxima over the accumulated set
                    float mx[GP];
#pragma unroll
                    for (int g = 0; g < GP; ++g) mx[g] = kNegInf;
                    for (int j = tid; j < nc; j += NT)
                        if (!m.sel[j]) {
#pragma unroll
                            for (int g = 0; g < GP; ++g) mx[g] = fmaxf(mx[g], m.S[(size_t)j * RS + g0 + g]);
                        }
#pragma unroll
                    for (int g = 0; g < GP; ++g) {
                        const float w = warp_max(mx[g]);
                        if (lane == 0) m.red[warp * GPAD + g0 + g] = w;
                    }
                }
                __syncthreads();
                for (int g = tid; g < GPAD; g += NT) {
                    float w = m.red[g];
                    for (int i = 1; i < NT / 32; ++i) w = fmaxf(w, m.red[i * GPAD + g]);
                    lm[g] = w;
                }
                __syncthreads();
                for (int g0 = 0; g0 < GPAD; g0 += GP) {   // probabilities in place, row sums
                    float sm[GP];
#pragma unroll
                    for (int g = 0; g < GP; ++g) sm[g] = 0.f;
                    for (int j = tid; j < nc; j += NT) {
                        const bool keep = m.sel[j];
#pragma unroll
                        for (int g = 0; g < GP; ++g) {
                            float* sp = m.S + (size_t)j * RS + g0 + g;
                            const float pr = keep ? 0.f : expf(*sp - lm[g0 + g]);
                            *sp = pr;
                            sm[g] += pr;
                        }
                    }
#pragma unroll
                    for (int g = 0; g < GP; ++g) {
                        const float w = warp_sum(sm[g]);
                        if (lane == 0) m.red[warp * GPAD + g0 + g] = w;
                    }
                }
                __syncthreads();
                for (int g = tid; g < GPAD; g += NT) {
                    float w = 0.f;
                    for (int i = 0; i < NT / 32; ++i) w += m.red[i * GPAD + g];
                    ls[g] = w;
                }
                // out[g][d] = sum_j p[j][g] * V[node_j][d]: thread = (candidate slice, value column)
                const int vcols = V < NT ? V : NT;
                const int nsl = NT / vcols;
                const int slice = tid / vcols, dcol = tid - slice * vcols;
                for (int g0 = 0; g0 < GPAD; g0 += GP) {
                    for (int d0 = 0; d0 < V; d0 += vcols) {
                        const int d = d0 + dcol;
                        float acc[GP];
#pragma unroll
                        for (int g = 0; g < GP; ++g) acc[g] = 0.f;
                        if (slice < nsl && d < V) {
                            for (int j = slice; j < nc; j += nsl) {
                                if (m.sel[j]) continue;
                                int node = par[j / CR] * CR + j % CR;
                                if (node < 0 || node >= Nl) node = 0;
                                const float vv = to_f(lv[(((int64_t)b * Nl + node) * p.Hkv + hk) * V + d]);
                                const float* pr = m.S + (size_t)j * RS + g0;
#pragma unroll
                                for (int g = 0; g < GP; g += 4) {
                                    const float4 x = *reinterpret_cast<const float4*>(pr + g);
                                    acc[g] += x.x * vv; acc[g + 1] += x.y * vv; acc[g + 2] += x.z * vv; acc[g + 3] += x.w * vv;
                                }
                            }
                        }
#pragma unroll
                        for (int g = 0; g < GP; ++g) m.part[tid * GP + g] = acc[g];
                        __syncthreads();
                        for (int i = tid; i < GP * vcols; i += NT) {
                            const int g = i / vcols, dc = i - g * vcols;
                            if (d0 + dc < V) {
                                float w = 0.f;
                                for (int s2 = 0; s2 < nsl; ++s2) w += m.part[(s2 * vcols + dc) * GP + g];
                                m.lo[(g0 + g) * V + d0 + dc] = w;
                            }
                        }
                        __syncthreads();
                    }
                }
            } else {
                for (int g = tid; g < GPAD; g += NT) { lm[g] = kNegInf; ls[g] = 0.f; }
                for (int i = tid; i < GPAD * V; i += NT) m.lo[i] = 0.f;
                __syncthreads();
            }

            // ---- trace + 5. merge into the running state (src/naive.py:215-223) ----
            if (p.tr_max) for (int g = tid; g < G; g += NT) p.tr_max[tslot * p.B * p.Tq * p.H + hbase + g] = lm[g];
            if (p.tr_sum) for (int g = tid; g < G; g += NT) p.tr_sum[tslot * p.B * p.Tq * p.H + hbase + g] = ls[g];
            if (p.tr_out)
                for (int i = tid; i < G * V; i += NT)
                    p.tr_out[(tslot * p.B * p.Tq * p.H + hbase) * V + i] = m.lo[i];
            for (int g = tid; g < GPAD; g += NT) {
                const bool ch = ls[g] > kHasMass, gh = gs[g] > kHasMass;
                const float nm = fmaxf(gm[g], lm[g]);
                sg[g] = gh ? expf(gm[g] - nm) : 0.f;
                sc[g] = ch ? expf(lm[g] - nm) : 0.f;
            }
            __syncthreads();
            for (int i = tid; i < GPAD * V; i += NT) {
                const int g = i / V;
                const bool ch = ls[g] > kHasMass, gh = gs[g] > kHasMass;
                if (ch) m.gout[i] = gh ? m.gout[i] * sg[g] + m.lo[i] * sc[g] : m.lo[i];
            }
            __syncthreads();
            for (int g = tid; g < GPAD; g += NT) {
                const bool ch = ls[g] > kHasMass, gh = gs[g] > kHasMass;
                if (ch) {
                    gs[g] = gh ? gs[g] * sg[g] + ls[g] * sc[g] : ls[g];
                    gm[g] = gh ? fmaxf(gm[g], lm[g]) : lm[g];
                }
            }
        }
        __syncthreads();
        if (p.level_mode && l > 0 && p.next_out) for (int i = tid; i < TK; i += NT) p.next_out[qidx * TK + i] = nxt[i];
        int32_t* tmp = par; par = nxt; nxt = tmp;   // the kept nodes are the next level's parents
        if (l == 0) { tmp = par; par = nxt; nxt = tmp; }
    }

    if (!select_only && !p.level_mode) {
        T* og = reinterpret_cast<T*>(p.out) + hbase * V;
        for (int i = tid; i < G * V; i += NT) og[i] = from_f<T>(m.gout[i] / gs[i / V]);   // src/parallel.py:321-363
        for (int g = tid; g < G; g += NT) { p.gmax[hbase + g] = gm[g]; p.gsum[hbase + g] = gs[g]; }
    }
}

template <typename T, bool TILED>
static int launch_tt(const AttnParams& p, size_t smem, int GP, cudaStream_t st) {
    dim3 grid(p.Tq, p.B * p.Hkv);
    cudaError_t e;
#define HT_LAUNCH(GPV)                                                                                                     \
    e = cudaFuncSetAttribute(fwd_generic_kernel<T, GPV, TILED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return (int)e;                                                                                   \
    fwd_generic_kernel<T, GPV, TILED><<<grid, NT, smem, st>>>(p);
    if (GP == 4) { HT_LAUNCH(4) } else if (GP == 8) { HT_LAUNCH(8) } else { HT_LAUNCH(16) }
#undef HT_LAUNCH
    note_launch();
    return (int)cudaGetLastError();
}

template <typename T>
static int launch_t(const AttnParams& p, cudaStream_t st) {
    const int G = p.G;
    const int GP = G <= 4 ? 4 : (G <= 8 ? 8 : 16);
    const int GPAD = (G + GP - 1) / GP * GP;
    const size_t limit = 227 * 1024;
    const size_t full = fwd_smem_layout(p.K, p.V, GPAD, GP, p.TK * p.CR, p.TK, false, nullptr, nullptr);
    if (full <= limit && !(p.flags & HTREE_FWD_TILED)) return launch_tt<T, false>(p, full, GP, st);
    const size_t tiled = fwd_smem_layout(p.K, p.V, GPAD, GP, p.TK * p.CR, p.TK, true, nullptr, nullptr);
    if (tiled > limit) return HTREE_E_UNSUPPORTED;
    return launch_tt<T, true>(p, tiled, GP, st);
}

// Stand-alone level merge and final normalisation: the reference's htree_merge_to_global_kernel and
// htree_final_normalize_kernel (src/parallel.py:248-363), kept for callers that drive the levels one by one.  One warp
// per (b, t, h) row.  The fused kernels do this on chip.
__global__ void __launch_bounds__(256) merge_to_global_kernel(const float* lmax, const float* lsum, const float* lout, float* gmax,
                                                              float* gsum, float* gout, int64_t rows, int V) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float lm = lmax[row], ls = lsum[row], gm = gmax[row], gs = gsum[row];
    const bool ch = ls > kHasMass, gh = gs > kHasMass;
    if (!ch) return;
    const float nm = fmaxf(gm, lm);
    const float sg = gh ? expf(gm - nm) : 0.f, sc = expf(lm - nm);
    for (int d = lane; d < V; d += 32) {
        const float o = lout[row * V + d];
        gout[row * V + d] = gh ? gout[row * V + d] * sg + o * sc : o;
    }
    __syncwarp();
    if (lane == 0) { gmax[row] = gh ? nm : lm; gsum[row] = gh ? gs * sg + ls * sc : ls; }
}

template <typename T>
__global__ void __launch_bounds__(256) final_normalize_kernel(const float* gout, const float* gsum, T* out, int64_t rows, int V) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * V) return;
    out[i] = from_f<T>(gout[i] / gsum[i / V]);
}

int launch_merge_to_global(const float* lmax, const float* lsum, const float* lout, float* gmax, float* gsum, float* gout,
                           int64_t rows, int V, cudaStream_t st) {
    merge_to_global_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(lmax, lsum, lout, gmax, gsum, gout, rows, V);
    note_launch();
    return (int)cudaGetLastError();
}

int launch_final_normalize(const float* gout, const float* gsum, void* out, int dtype, int64_t rows, int V, cudaStream_t st) {
    const unsigned blocks = (unsigned)((rows * V + 255) / 256);
    if (dtype == HTREE_F32) final_normalize_kernel<float><<<blocks, 256, 0, st>>>(gout, gsum, (float*)out, rows, V);
    else if (dtype == HTREE_BF16) final_normalize_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(gout, gsum, (__nv_bfloat16*)out, rows, V);
    else final_normalize_kernel<__half><<<blocks, 256, 0, st>>>(gout, gsum, (__half*)out, rows, V);
    note_launch();
    return (int)cudaGetLastError();
}

int launch_fwd_generic(const AttnParams& p, int dtype, cudaStream_t st) {
    switch (dtype) {
        case HTREE_F32: return launch_t<float>(p, st);
        case HTREE_BF16: return launch_t<__nv_bfloat16>(p, st);
        default: return launch_t<__half>(p, st);
    }
}

}  // namespace htree
