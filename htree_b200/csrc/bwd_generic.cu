// Storage-type-generic backward: one thread block per (batch, query position, KV head, chunk of <= 16 query heads),
// fp32 arithmetic, all levels in one launch.
//
// Behaviour follows src/naive.py:333-386 (selections are constants); the reference's GPU kernels for the same work
// are htree_bwd_preprocess_delta_kernel, htree_bwd_dq_bottom/upper_kernel, htree_bwd_build_parent_mask_kernel and
// htree_bwd_dkv_bottom/upper_kernel (src/backward.py:45-780).  Differences by design:
//   * the row-sum D = sum_v dO*out is computed here, from out/dO in their storage type (no fp32 copies);
//   * dK/dV are reduced with fp32 atomic adds from this query-stationary pass instead of a dense
//     [B,H_kv,groups,T] byte mask scanned serially by key-stationary programs;
//   * dq is kept on chip across levels and written once.
// Per level: the accumulated set = candidates absent from the next level's parent list (binary search; both
// sorted).  For tiles of up to 256 accumulated candidates: (A) one thread per candidate recomputes S and
// dP = dO.V^T, forms P = exp(S-gmax)/gsum and dS = P*(dP-D) into shared memory; (B) threads re-map to
// (candidate slice, rotation pair) to accumulate dq~ += dS*k~ in registers and to push
// dK[node] += R^-1(sum_h dS*q~), and to (slice, value column) to push dV[node] += sum_h P*dO.
#include "common.cuh"

namespace htree {

constexpr int NTB = 256;

struct BwdSmem {
    float* qT;     // [K][GP]  rotated, scaled queries of this head chunk
    float* dOT;    // [V][GP]
    float* dqT;    // [K][GP]  level reduction of dq~
    float* dqs;    // [GP][K]  dq summed over levels
    float* Pt;     // [NTB][GP+4]
    float* dSt;    // [NTB][GP+4]
    float* hd;     // D, gmax, gsum: 3 x [GP]
    int32_t* par;  // [TK]
    int32_t* nsel; // [TK]
    uint16_t* ul;  // [maxc]  positions of the accumulated candidates
    int* wtot;     // [NTB/32]
};

__host__ __device__ inline size_t bwd_smem_layout(int K, int V, int GP, int maxc, int TK, BwdSmem* m, unsigned char* base) {
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t r = o; o = (o + bytes + 15) & ~size_t(15); return r; };
    size_t a0 = take(sizeof(float) * K * GP), a1 = take(sizeof(float) * V * GP), a2 = take(sizeof(float) * K * GP);
    size_t a3 = take(sizeof(float) * GP * K), a4 = take(sizeof(float) * NTB * (GP + 4)), a5 = take(sizeof(float) * NTB * (GP + 4));
    size_t a6 = take(sizeof(float) * 3 * GP), a7 = take(sizeof(int32_t) * TK), a8 = take(sizeof(int32_t) * TK);
    size_t a9 = take(sizeof(uint16_t) * maxc), a10 = take(sizeof(int) * (NTB / 32));
    if (m) {
        m->qT = (float*)(base + a0); m->dOT = (float*)(base + a1); m->dqT = (float*)(base + a2); m->dqs = (float*)(base + a3);
        m->Pt = (float*)(base + a4); m->dSt = (float*)(base + a5); m->hd = (float*)(base + a6);
        m->par = (int32_t*)(base + a7); m->nsel = (int32_t*)(base + a8); m->ul = (uint16_t*)(base + a9); m->wtot = (int*)(base + a10);
    }
    return o;
}

template <typename T, int GP>
__global__ void __launch_bounds__(NTB) bwd_generic_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, V = p.V, CR = p.CR, TK = p.TK, L = p.L, half = K >> 1;
    constexpr int RS = GP + 4;
    BwdSmem m;
    bwd_smem_layout(K, V, GP, TK * CR, TK, &m, smem_raw);
    float *Dg = m.hd, *gmx = m.hd + GP, *gsm = m.hd + 2 * GP;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = p.t0 + blockIdx.x;                                         // query window: row blockIdx.x is position t0 + blockIdx.x
    const int b = blockIdx.y / p.Hkv, hk = blockIdx.y % p.Hkv;
    const int g_begin = blockIdx.z * 16;
    const int Gc = min(16, p.G - g_begin);                                   // heads of this chunk
    const int64_t hbase = ((int64_t)b * p.Tq + blockIdx.x) * p.H + (int64_t)hk * p.G + g_begin;
    const int64_t qidx = ((int64_t)b * p.Tq + blockIdx.x) * p.Hkv + hk;
    const T* qg = reinterpret_cast<const T*>(p.q) + hbase * K;
    const T* dOg = reinterpret_cast<const T*>(p.dO) + hbase * V;
    const T* og = reinterpret_cast<const T*>(p.out) + hbase * V;

    // ---- per-query constants: dO (head-minor), D = sum_v dO*out, gmax, gsum ----
    for (int i = tid; i < GP * V; i += NTB) {
        const int g = i / V, d = i - g * V;
        m.dOT[d * GP + g] = g < Gc ? to_f(dOg[(int64_t)g * V + d]) : 0.f;
    }
    for (int i = tid; i < GP * K; i += NTB) m.dqs[i] = 0.f;
    for (int g = warp; g < GP; g += NTB / 32) {
        float s = 0.f;
        if (g < Gc) for (int d = lane; d < V; d += 32) s += to_f(dOg[(int64_t)g * V + d]) * to_f(og[(int64_t)g * V + d]);
        s = warp_sum(s);
        if (lane == 0) {
            Dg[g] = s;
            gmx[g] = g < Gc ? p.gmax[hbase + g] : 0.f;
            gsm[g] = g < Gc ? p.gsum[hbase + g] : 1.f;
        }
    }
    __syncthreads();

    const int nslB = NTB / half;                       // candidate slices of the (slice, pair) mapping
    const int sliceB = tid / half, pairB = tid - sliceB * half;
    const bool actB = sliceB < nslB;
    const int vcols = V < NTB ? V : NTB;
    const int nslV = NTB / vcols;
    const int sliceV = tid / vcols, dcolV = tid - sliceV * vcols;

    for (int l = L - 1; l >= 0; --l) {
        const int Nl = p.ln[l];
        const T* lk = reinterpret_cast<const T*>(p.lk[l]);
        const T* lv = reinterpret_cast<const T*>(p.lv[l]);
        float* dkl = p.dk[l];
        float* dvl = p.dv[l];
        for (int i = tid; i < TK; i += NTB) {
            m.par[i] = load_parent(p, l, qidx * TK + i);
            m.nsel[i] = l > 0 ? load_parent(p, l - 1, qidx * TK + i) : -1;
        }
        __syncthreads();
        int np = 0, nsv = 0;
        for (int i = tid; i < TK; i += NTB) { np += m.par[i] >= 0; nsv += m.nsel[i] >= 0; }
        np = __reduce_add_sync(0xffffffffu, np);
        nsv = __reduce_add_sync(0xffffffffu, nsv);
        if (lane == 0) m.wtot[warp] = np | (nsv << 16);
        __syncthreads();
        np = 0; nsv = 0;
#pragma unroll
        for (int i = 0; i < NTB / 32; ++i) { np += m.wtot[i] & 0xffff; nsv += m.wtot[i] >> 16; }
        __syncthreads();
        if (np <= 0) continue;
        const int rci = (int)(((int64_t)t / p.lpow[l]) % CR);
        const int nc = (np - 1) * CR + rci + 1, rp = nc - 1;

        // queries of this chunk, rotated to the right-most position and scaled
        for (int i = tid; i < GP * half; i += NTB) {
            const int g = i / half, d = i - g * half;
            float a = 0.f, c = 0.f;
            if (g < Gc) {
                const float lo = to_f(qg[(int64_t)g * K + d]), hi = to_f(qg[(int64_t)g * K + d + half]);
                const float cs = __ldg(p.cosc + (int64_t)rp * half + d), sn = __ldg(p.sinc + (int64_t)rp * half + d);
                a = (lo * cs - hi * sn) * p.scale;
                c = (lo * sn + hi * cs) * p.scale;
            }
            m.qT[d * GP + g] = a;
            m.qT[(d + half) * GP + g] = c;
        }
        // accumulated set: ordered compaction of the candidates that the next level did not keep
        int nu = 0;
        for (int j0 = 0; j0 < nc; j0 += NTB) {
            const int j = j0 + tid;
            bool f = j < nc;
            if (f && l > 0) {
                const int node = m.par[j / CR] * CR + j % CR;
                int lo = 0, hi = nsv;
                while (lo < hi) { const int mid = (lo + hi) >> 1; if (m.nsel[mid] < node) lo = mid + 1; else hi = mid; }
                f = !(lo < nsv && m.nsel[lo] == node);
            }
            int tot;
            const int pos = nu + block_scan_flag<NTB>(f, m.wtot, &tot);
            if (f) m.ul[pos] = (uint16_t)j;
            nu += tot;
        }
        __syncthreads();

        float dqlo[GP], dqhi[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) { dqlo[g] = 0.f; dqhi[g] = 0.f; }

        for (int u0 = 0; u0 < nu; u0 += NTB) {
            const int tn = min(NTB, nu - u0);
            // ---- (A) one accumulated candidate per thread: S, dP -> P, dS ----
            {
                float P[GP], dS[GP];
#pragma unroll
                for (int g = 0; g < GP; ++g) { P[g] = 0.f; dS[g] = 0.f; }
                if (tid < tn) {
                    const int j = m.ul[u0 + tid];
                    int node = m.par[j / CR] * CR + j % CR;
                    if (node < 0 || node >= Nl) { if (p.status) atomicOr(p.status, 2); node = 0; }
                    const T* kr = lk + (((int64_t)b * Nl + node) * p.Hkv + hk) * K;
                    const T* vr = lv + (((int64_t)b * Nl + node) * p.Hkv + hk) * V;
                    const float* cj = p.cosc + (int64_t)j * half;
                    const float* sj = p.sinc + (int64_t)j * half;
                    float S[GP], dP[GP];
#pragma unroll
                    for (int g = 0; g < GP; ++g) { S[g] = 0.f; dP[g] = 0.f; }
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
                            const float* qa = m.qT + (d + u) * GP;
                            const float* qb = m.qT + (d + u + half) * GP;
#pragma unroll
                            for (int g = 0; g < GP; g += 4) {
                                const float4 x = *reinterpret_cast<const float4*>(qa + g);
                                const float4 y = *reinterpret_cast<const float4*>(qb + g);
                                S[g] += x.x * klo; S[g + 1] += x.y * klo; S[g + 2] += x.z * klo; S[g + 3] += x.w * klo;
                                S[g] += y.x * khi; S[g + 1] += y.y * khi; S[g + 2] += y.z * khi; S[g + 3] += y.w * khi;
                            }
                        }
                    }
                    for (int d = 0; d < V; d += 4) {
                        float vv[4];
                        load4<T>(vr + d, vv);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float* da = m.dOT + (d + u) * GP;
#pragma unroll
                            for (int g = 0; g < GP; g += 4) {
                                const float4 x = *reinterpret_cast<const float4*>(da + g);
                                dP[g] += x.x * vv[u]; dP[g + 1] += x.y * vv[u]; dP[g + 2] += x.z * vv[u]; dP[g + 3] += x.w * vv[u];
                            }
                        }
                    }
#pragma unroll
                    for (int g = 0; g < GP; ++g) {
                        if (g < Gc) {
                            P[g] = expf(S[g] - gmx[g]) / gsm[g];          // src/naive.py:379
                            dS[g] = P[g] * (dP[g] - Dg[g]);               // src/naive.py:382
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < GP; g += 4) {
                    *reinterpret_cast<float4*>(m.Pt + tid * RS + g) = make_float4(P[g], P[g + 1], P[g + 2], P[g + 3]);
                    *reinterpret_cast<float4*>(m.dSt + tid * RS + g) = make_float4(dS[g], dS[g + 1], dS[g + 2], dS[g + 3]);
                }
            }
            __syncthreads();
            // ---- (B1) dq~ and dK: thread = (candidate slice, rotation pair) ----
            if (actB) {
                float qlo[GP], qhi[GP];
#pragma unroll
                for (int g = 0; g < GP; ++g) { qlo[g] = m.qT[pairB * GP + g]; qhi[g] = m.qT[(pairB + half) * GP + g]; }
                for (int u = sliceB; u < tn; u += nslB) {
                    const int j = m.ul[u0 + u];
                    int node = m.par[j / CR] * CR + j % CR;
                    if (node < 0 || node >= Nl) node = 0;
                    const int64_t row = (((int64_t)b * Nl + node) * p.Hkv + hk) * K;
                    const float lo = to_f(lk[row + pairB]), hi = to_f(lk[row + pairB + half]);
                    const float cs = __ldg(p.cosc + (int64_t)j * half + pairB), sn = __ldg(p.sinc + (int64_t)j * half + pairB);
                    const float klo = lo * cs - hi * sn, khi = lo * sn + hi * cs;
                    float dklo = 0.f, dkhi = 0.f;
                    const float* ds = m.dSt + u * RS;
#pragma unroll
                    for (int g = 0; g < GP; g += 4) {
                        const float4 x = *reinterpret_cast<const float4*>(ds + g);
                        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            dqlo[g + w] += xs[w] * klo; dqhi[g + w] += xs[w] * khi;
                            dklo += xs[w] * qlo[g + w]; dkhi += xs[w] * qhi[g + w];
                        }
                    }
                    atomicAdd(dkl + row + pairB, dklo * cs + dkhi * sn);               // inverse rotation, src/naive.py:31-38
                    atomicAdd(dkl + row + pairB + half, -dklo * sn + dkhi * cs);
                }
            }
            // ---- (B2) dV: thread = (candidate slice, value column) ----
            if (sliceV < nslV) {
                for (int d0 = 0; d0 < V; d0 += vcols) {
                    const int d = d0 + dcolV;
                    if (d >= V) break;
                    float dcol[GP];
#pragma unroll
                    for (int g = 0; g < GP; ++g) dcol[g] = m.dOT[d * GP + g];
                    for (int u = sliceV; u < tn; u += nslV) {
                        const int j = m.ul[u0 + u];
                        int node = m.par[j / CR] * CR + j % CR;
                        if (node < 0 || node >= Nl) node = 0;
                        const float* pr = m.Pt + u * RS;
                        float acc = 0.f;
#pragma unroll
                        for (int g = 0; g < GP; g += 4) {
                            const float4 x = *reinterpret_cast<const float4*>(pr + g);
                            acc += x.x * dcol[g] + x.y * dcol[g + 1] + x.z * dcol[g + 2] + x.w * dcol[g + 3];
                        }
                        atomicAdd(dvl + (((int64_t)b * Nl + node) * p.Hkv + hk) * V + d, acc);   // src/naive.py:386
                    }
                }
            }
            __syncthreads();
        }

        // ---- level reduction of dq~ over the candidate slices, inverse rotation, running sum ----
        for (int s = 0; s < nslB; ++s) {
            if (actB && sliceB == s) {
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                    if (s == 0) { m.dqT[pairB * GP + g] = dqlo[g]; m.dqT[(pairB + half) * GP + g] = dqhi[g]; }
                    else { m.dqT[pairB * GP + g] += dqlo[g]; m.dqT[(pairB + half) * GP + g] += dqhi[g]; }
                }
            }
            __syncthreads();
        }
        for (int i = tid; i < GP * half; i += NTB) {
            const int g = i / half, d = i - g * half;
            const float lo = m.dqT[d * GP + g], hi = m.dqT[(d + half) * GP + g];
            const float cs = __ldg(p.cosc + (int64_t)rp * half + d), sn = __ldg(p.sinc + (int64_t)rp * half + d);
            m.dqs[g * K + d] += p.scale * (lo * cs + hi * sn);                           // src/naive.py:384
            m.dqs[g * K + d + half] += p.scale * (-lo * sn + hi * cs);
        }
        __syncthreads();
    }
    if (p.dq_typed) {   // rounded once to the storage type instead of an fp32 tensor the caller casts afterwards
        T* dqt = reinterpret_cast<T*>(p.dq_typed);
        for (int i = tid; i < Gc * K; i += NTB) dqt[hbase * K + i] = from_f<T>(m.dqs[i]);
    } else {
        for (int i = tid; i < Gc * K; i += NTB) p.dq[hbase * K + i] = m.dqs[i];
    }
}

template <typename T>
static int launch_bt(const AttnParams& p, cudaStream_t st) {
    const int Gc = p.G < 16 ? p.G : 16;
    const int GP = Gc <= 4 ? 4 : (Gc <= 8 ? 8 : 16);
    if (p.K / 2 > NTB || p.TK * p.CR > 65535) return HTREE_E_UNSUPPORTED;
    const size_t smem = bwd_smem_layout(p.K, p.V, GP, p.TK * p.CR, p.TK, nullptr, nullptr);
    if (smem > 227 * 1024) return HTREE_E_UNSUPPORTED;
    dim3 grid(p.Tq, p.B * p.Hkv, (p.G + 15) / 16);
    cudaError_t e;
#define HT_LAUNCH(GPV)                                                                                              \
    e = cudaFuncSetAttribute(bwd_generic_kernel<T, GPV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return (int)e;                                                                            \
    bwd_generic_kernel<T, GPV><<<grid, NTB, smem, st>>>(p);
    if (GP == 4) { HT_LAUNCH(4) } else if (GP == 8) { HT_LAUNCH(8) } else { HT_LAUNCH(16) }
#undef HT_LAUNCH
    note_launch();
    return (int)cudaGetLastError();
}

// The size checks of the launcher, for callers that must decide before they queue any work.
bool bwd_generic_supported(const AttnParams& p, int dtype) {
    (void)dtype;
    const int Gc = p.G < 16 ? p.G : 16;
    const int GP = Gc <= 4 ? 4 : (Gc <= 8 ? 8 : 16);
    if (p.K / 2 > NTB || p.TK * p.CR > 65535) return false;
    return bwd_smem_layout(p.K, p.V, GP, p.TK * p.CR, p.TK, nullptr, nullptr) <= 227 * 1024;
}

int launch_bwd_generic(const AttnParams& p, int dtype, cudaStream_t st) {
    switch (dtype) {
        case HTREE_F32: return launch_bt<float>(p, st);
        case HTREE_BF16: return launch_bt<__nv_bfloat16>(p, st);
        default: return launch_bt<__half>(p, st);
    }
}

}  // namespace htree
