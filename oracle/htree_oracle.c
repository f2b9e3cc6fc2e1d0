/*
 * CPU oracle for htree hierarchical tree sparse attention.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's loop oracle (src/naive.py in skywong14/htree), evaluated one
 * (batch, query position, KV head) group at a time so that sampled queries of very long sequences can be checked.
 * Nothing in the shipped CUDA path calls into this file; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark do.
 *
 * Parity pin: the outputs of this file are compared with tensors produced by the reference's own
 * htree_forward_naive / HTreeFunction on seeded inputs (tests/golden/).
 *
 * All arrays are float32 and contiguous.  Inputs whose storage type is bf16/fp16 are passed as float32 arrays that
 * hold exactly representable values; ho_round() performs the round-to-nearest-even storage rounding where the
 * reference stores a tensor in the input dtype (pooled tree levels, the final output, the returned gradients).
 *
 * Layouts (reference: src/naive.py:143-147):  q [B,T,H,K]  k [B,N_l,H_kv,K]  v [B,N_l,H_kv,V]  out [B,T,H,V].
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HO_NEG_INF (-1.0e10f) /* src/naive.py:9 */

typedef struct {
    int32_t B, T, H, H_kv, K, V;
    int32_t CR;        /* compression_rate */
    int32_t TK;        /* top_k_per_layer */
    int32_t L;         /* number of tree levels, level 0 = leaves */
    int32_t n_pos;     /* rows of the cos/sin tables */
    float scale;
} HoShape;

/* ---- storage rounding -------------------------------------------------------------------------------------- */

static float round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x; /* inf / nan unchanged */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}

static float round_fp16(float x) {
    /* round-to-nearest-even to IEEE half, returned as float (handles subnormals and overflow to inf) */
    if (!(x == x) || isinf(x)) return x;
    float ax = fabsf(x);
    if (ax >= 65520.0f) return x > 0 ? INFINITY : -INFINITY;
    if (ax < 6.103515625e-05f) { /* subnormal half: spacing 2^-24 */
        float r = nearbyintf(ax * 16777216.0f) / 16777216.0f;
        return x < 0 ? -r : r;
    }
    int e;
    frexpf(ax, &e);                      /* ax = m * 2^e, m in [0.5,1) */
    float ulp = ldexpf(1.0f, e - 11);    /* 11 significant bits */
    float r = nearbyintf(ax / ulp) * ulp;
    return x < 0 ? -r : r;
}

/* dtype: 0 = float32 (no-op), 1 = bfloat16, 2 = float16 */
void ho_round(float* x, int64_t n, int dtype) {
    if (dtype == 1) for (int64_t i = 0; i < n; ++i) x[i] = round_bf16(x[i]);
    else if (dtype == 2) for (int64_t i = 0; i < n; ++i) x[i] = round_fp16(x[i]);
}

/* ---- tree --------------------------------------------------------------------------------------------------- */

/* Number of levels: keep pooling while the level is longer than max_top_nodes (src/naive.py:49-59). */
int ho_num_levels(int T, int CR, int MTN) {
    int L = 1, n = T;
    while (n > MTN) { n = (n + CR - 1) / CR; ++L; }
    return L;
}

/* One pooling step, parent = mean of its valid children, stored in the input dtype (src/naive.py:53-57). */
void ho_build_level(const float* child, float* parent, int B, int Nc, int Hkv, int D, int CR, int dtype) {
    int Np = (Nc + CR - 1) / CR;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int p = 0; p < Np; ++p) {
            int s = p * CR, e = s + CR < Nc ? s + CR : Nc;
            for (int h = 0; h < Hkv; ++h)
                for (int d = 0; d < D; ++d) {
                    float acc = 0.f;
                    for (int c = s; c < e; ++c) acc += child[(((int64_t)b * Nc + c) * Hkv + h) * D + d];
                    float m = acc / (float)(e - s);
                    if (dtype == 1) m = round_bf16(m); else if (dtype == 2) m = round_fp16(m);
                    parent[(((int64_t)b * Np + p) * Hkv + h) * D + d] = m;
                }
        }
}

/* Mean-pool gradient, parent level -> child level: child += parent / count (src/naive.py:388-394). */
void ho_tree_backward_level(const float* dparent, float* dchild, int B, int Nc, int Hkv, int D, int CR) {
    int Np = (Nc + CR - 1) / CR;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int p = 0; p < Np; ++p) {
            int s = p * CR, e = s + CR < Nc ? s + CR : Nc;
            float cnt = (float)(e - s);
            for (int c = s; c < e; ++c)
                for (int64_t x = 0; x < (int64_t)Hkv * D; ++x)
                    dchild[((int64_t)b * Nc + c) * Hkv * D + x] += dparent[((int64_t)b * Np + p) * Hkv * D + x] / cnt;
        }
}

/* ---- per-group forward ------------------------------------------------------------------------------------ */

static inline void rope_fwd(const float* x, const float* c, const float* s, float* y, int K) {
    int half = K / 2; /* src/naive.py:22-28: half-split rotation */
    for (int i = 0; i < half; ++i) {
        float lo = x[i], hi = x[i + half];
        y[i] = lo * c[i] - hi * s[i];
        y[i + half] = lo * s[i] + hi * c[i];
    }
}

static inline void rope_inv(const float* x, const float* c, const float* s, float* y, int K) {
    int half = K / 2; /* src/naive.py:31-38 */
    for (int i = 0; i < half; ++i) {
        float lo = x[i], hi = x[i + half];
        y[i] = lo * c[i] + hi * s[i];
        y[i + half] = -lo * s[i] + hi * c[i];
    }
}

typedef struct { float imp; int32_t pos; } ImpPos;

static int cmp_imp_desc_stable(const void* a, const void* b) {
    const ImpPos* x = (const ImpPos*)a; const ImpPos* y = (const ImpPos*)b;
    if (x->imp > y->imp) return -1;
    if (x->imp < y->imp) return 1;
    return x->pos < y->pos ? -1 : (x->pos > y->pos ? 1 : 0); /* stable: ties keep the smaller position first */
}

/* Scratch for one group. */
typedef struct {
    float *qr, *kr, *S, *imp, *lo, *gout, *tmpk;
    int32_t *par, *npar, *node;
    uint8_t* sel;
    ImpPos* order;
} Scratch;

static int scratch_alloc(Scratch* w, const HoShape* sh) {
    int G = sh->H / sh->H_kv, maxc = sh->TK * sh->CR;
    w->qr = (float*)malloc(sizeof(float) * G * sh->K);
    w->kr = (float*)malloc(sizeof(float) * (size_t)maxc * sh->K);
    w->S = (float*)malloc(sizeof(float) * (size_t)G * maxc);
    w->imp = (float*)malloc(sizeof(float) * maxc);
    w->lo = (float*)malloc(sizeof(float) * G * sh->V);
    w->gout = (float*)malloc(sizeof(float) * G * sh->V);
    w->tmpk = (float*)malloc(sizeof(float) * sh->K);
    w->par = (int32_t*)malloc(sizeof(int32_t) * sh->TK);
    w->npar = (int32_t*)malloc(sizeof(int32_t) * sh->TK);
    w->node = (int32_t*)malloc(sizeof(int32_t) * maxc);
    w->sel = (uint8_t*)malloc(maxc);
    w->order = (ImpPos*)malloc(sizeof(ImpPos) * maxc);
    return w->qr && w->kr && w->S && w->imp && w->lo && w->gout && w->tmpk && w->par && w->npar && w->node && w->sel && w->order;
}

static void scratch_free(Scratch* w) {
    free(w->qr); free(w->kr); free(w->S); free(w->imp); free(w->lo); free(w->gout); free(w->tmpk);
    free(w->par); free(w->npar); free(w->node); free(w->sel); free(w->order);
}

static int64_t ipow(int64_t b, int e) { int64_t r = 1; while (e-- > 0) r *= b; return r; }

/*
 * Forward for a list of groups (b, t, h_kv).  Follows src/naive.py:171-231 for each group.
 *
 *   queries   [nq,3] int32 (b,t,h_kv), or NULL meaning every group in (b,t,h_kv) row-major order (nq = B*T*H_kv)
 *   out       [nq,G,V]  un-rounded fp32 output  (g_out / g_sum)
 *   gmax,gsum [nq,G]
 *   parents   [L,nq,TK] int32 or NULL: parents[l] = the parent list CONSUMED at level l, ascending, -1 padded
 *             (the reference's per_layer_parents, src/naive.py:258)
 *   tr_max,tr_sum [L,nq,G], tr_out [L,nq,G,V] or NULL: per-level accumulator state (LayerTrace, src/naive.py:13-19)
 *   gap       [L,nq] or NULL: relative gap (imp_TK - imp_{TK+1}) / imp_TK between the last kept and the first
 *             dropped importance at levels that drop something, else +inf.  Used to classify near-ties.
 *   imp_out   [L,nq,TK*CR] or NULL: shared importance of every candidate position at the upper levels (right-most
 *             forced to 1e6), -1 where there is no candidate and at the leaf level.
 * Returns 0, or -1 on allocation failure, -2 if a node index leaves its level, -3 if a position leaves the tables.
 */
int ho_forward(const HoShape* sh, const float* q, const float* const* layers_k, const float* const* layers_v,
               const int32_t* level_n, const float* cosc, const float* sinc, const int32_t* queries, int64_t nq,
               float* out, float* gmax, float* gsum, int32_t* parents, float* tr_max, float* tr_sum, float* tr_out,
               float* gap, float* imp_out) {
    const int G = sh->H / sh->H_kv, K = sh->K, V = sh->V, CR = sh->CR, TK = sh->TK, L = sh->L, half = K / 2;
    const int64_t maxc = (int64_t)TK * CR;
    int status = 0;
    #pragma omp parallel
    {
        Scratch w;
        int ok = scratch_alloc(&w, sh);
        if (!ok) {
            #pragma omp atomic write
            status = -1;
        }
        #pragma omp barrier
        if (status == 0) {
        #pragma omp for schedule(dynamic, 8)
        for (int64_t qi = 0; qi < nq; ++qi) {
            int b, t, hk;
            if (queries) { b = queries[3 * qi]; t = queries[3 * qi + 1]; hk = queries[3 * qi + 2]; }
            else { hk = (int)(qi % sh->H_kv); t = (int)((qi / sh->H_kv) % sh->T); b = (int)(qi / ((int64_t)sh->H_kv * sh->T)); }
            const float* qg = q + (((int64_t)b * sh->T + t) * sh->H + (int64_t)hk * G) * K;
            float gm[64], gs[64];
            for (int g = 0; g < G; ++g) { gm[g] = HO_NEG_INF; gs[g] = 0.f; }
            memset(w.gout, 0, sizeof(float) * G * V);

            /* virtual parents of the top level (src/naive.py:108-118) */
            int np = (int)((t / ipow(CR, L - 1)) / CR) + 1;
            if (np > TK) np = TK;
            for (int i = 0; i < TK; ++i) w.par[i] = i < np ? i : -1;

            for (int l = L - 1; l >= 0; --l) {
                const int Nl = level_n[l];
                const float* lk = layers_k[l]; const float* lv = layers_v[l];
                if (parents) memcpy(parents + ((int64_t)l * nq + qi) * TK, w.par, sizeof(int32_t) * TK);
                np = 0; while (np < TK && w.par[np] >= 0) ++np;
                int rci = (int)((t / ipow(CR, l)) % CR);
                int nc = (np - 1) * CR + rci + 1, rp = nc - 1;
                if (nc < 1 || rp >= sh->n_pos) { status = -3; continue; }
                /* rotated, scaled queries (src/naive.py:197-198) */
                for (int g = 0; g < G; ++g) {
                    rope_fwd(qg + (int64_t)g * K, cosc + (int64_t)rp * half, sinc + (int64_t)rp * half, w.qr + g * K, K);
                    for (int d = 0; d < K; ++d) w.qr[g * K + d] *= sh->scale;
                }
                float lmax_all = -INFINITY;
                for (int j = 0; j < nc; ++j) {
                    int node = w.par[j / CR] * CR + j % CR; /* src/naive.py:188-190 */
                    if (node < 0 || node >= Nl) { status = -2; node = 0; }
                    w.node[j] = node;
                    const float* kn = lk + (((int64_t)b * Nl + node) * sh->H_kv + hk) * K;
                    rope_fwd(kn, cosc + (int64_t)j * half, sinc + (int64_t)j * half, w.kr + (int64_t)j * K, K);
                    for (int g = 0; g < G; ++g) {
                        float acc = 0.f;
                        const float* a = w.qr + g * K; const float* kk = w.kr + (int64_t)j * K;
                        for (int d = 0; d < K; ++d) acc += a[d] * kk[d];
                        w.S[(int64_t)g * nc + j] = acc;
                        if (acc > lmax_all) lmax_all = acc;
                    }
                }
                float gapv = INFINITY;
                if (l == 0) {
                    memset(w.sel, 0, (size_t)nc);
                } else {
                    /* shared importance and Top-K (src/naive.py:204-206, 88-105) */
                    for (int j = 0; j < nc; ++j) {
                        float s = 0.f;
                        for (int g = 0; g < G; ++g) s += expf(w.S[(int64_t)g * nc + j] - lmax_all);
                        w.imp[j] = s;
                    }
                    w.imp[rp] = 1e6f;
                    for (int j = 0; j < nc; ++j) { w.order[j].imp = w.imp[j]; w.order[j].pos = j; }
                    qsort(w.order, nc, sizeof(ImpPos), cmp_imp_desc_stable);
                    int take = TK < nc ? TK : nc;
                    memset(w.sel, 0, (size_t)nc);
                    for (int i = 0; i < take; ++i) w.sel[w.order[i].pos] = 1;
                    if (take < nc) gapv = (w.order[take - 1].imp - w.order[take].imp) / w.order[take - 1].imp;
                    int n = 0; /* node ids grow with the position, so position order is ascending node order */
                    for (int j = 0; j < nc; ++j) if (w.sel[j]) w.npar[n++] = w.node[j];
                    for (; n < TK; ++n) w.npar[n] = -1;
                }
                if (gap) gap[(int64_t)l * nq + qi] = gapv;
                if (imp_out) {
                    float* io = imp_out + ((int64_t)l * nq + qi) * maxc;
                    for (int64_t j = 0; j < maxc; ++j) io[j] = (l > 0 && j < nc) ? w.imp[j] : -1.f;
                }

                /* accumulate the unselected candidates (src/naive.py:73-85, 209-213) */
                float lm[64], ls[64];
                for (int g = 0; g < G; ++g) {
                    float m = HO_NEG_INF; int any = 0;
                    for (int j = 0; j < nc; ++j) if (!w.sel[j]) { any = 1; float s = w.S[(int64_t)g * nc + j]; if (s > m) m = s; }
                    float* o = w.lo + g * V;
                    memset(o, 0, sizeof(float) * V);
                    float sum = 0.f;
                    if (any) {
                        for (int j = 0; j < nc; ++j) if (!w.sel[j]) {
                            float p = expf(w.S[(int64_t)g * nc + j] - m);
                            sum += p;
                            const float* vn = lv + (((int64_t)b * Nl + w.node[j]) * sh->H_kv + hk) * V;
                            for (int d = 0; d < V; ++d) o[d] += p * vn[d];
                        }
                    }
                    lm[g] = m; ls[g] = sum;
                }
                if (tr_max) for (int g = 0; g < G; ++g) {
                    tr_max[((int64_t)l * nq + qi) * G + g] = lm[g];
                    tr_sum[((int64_t)l * nq + qi) * G + g] = ls[g];
                    memcpy(tr_out + (((int64_t)l * nq + qi) * G + g) * V, w.lo + g * V, sizeof(float) * V);
                }
                /* merge the level into the global state (src/naive.py:215-223) */
                for (int g = 0; g < G; ++g) {
                    int ch = ls[g] > 1e-10f, gh = gs[g] > 1e-10f;
                    float nm = gm[g] > lm[g] ? gm[g] : lm[g];
                    float sg = gh ? expf(gm[g] - nm) : 0.f;
                    float sc = ch ? expf(lm[g] - nm) : 0.f;
                    if (ch) {
                        float* go = w.gout + g * V; const float* o = w.lo + g * V;
                        if (gh) { for (int d = 0; d < V; ++d) go[d] = go[d] * sg + o[d] * sc; gs[g] = gs[g] * sg + ls[g] * sc; gm[g] = nm; }
                        else { memcpy(go, o, sizeof(float) * V); gs[g] = ls[g]; gm[g] = lm[g]; }
                    }
                }
                if (l > 0) memcpy(w.par, w.npar, sizeof(int32_t) * TK);
            }
            for (int g = 0; g < G; ++g) {
                gmax[qi * G + g] = gm[g]; gsum[qi * G + g] = gs[g];
                for (int d = 0; d < V; ++d) out[(qi * G + g) * V + d] = w.gout[g * V + d] / gs[g]; /* src/naive.py:231 */
            }
        }
        }
        scratch_free(&w);
    }
    return status;
}

/*
 * Backward for one group: adds into dk_layers/dv_layers (with atomics if `atomic`), writes dq [G,K].
 * Per-group arrays (out, dO, gmax, gsum, dq) are addressed by the flat group index qi; for the full tensors
 * [B,T,H,*] this is the same memory as [B*T*H_kv, G, *].
 */
static int backward_group(const HoShape* sh, const float* q, const float* const* layers_k, const float* const* layers_v,
                          const int32_t* level_n, const float* cosc, const float* sinc, const float* out,
                          const float* dO, const float* gmax, const float* gsum, const int32_t* parents, int64_t nq,
                          int64_t qi, int b, int t, int hk, float* dq, float* const* dk_layers, float* const* dv_layers,
                          int atomic, float* qr, float* kr, float* dqr, float* dkr, float* tmp, float* Dg) {
    const int G = sh->H / sh->H_kv, K = sh->K, V = sh->V, CR = sh->CR, TK = sh->TK, L = sh->L, half = K / 2;
    int status = 0;
    const float* qg = q + (((int64_t)b * sh->T + t) * sh->H + (int64_t)hk * G) * K;
    const int64_t hb = qi * G;
    for (int g = 0; g < G; ++g) { /* D = sum_v dO * out (src/naive.py:333) */
        float s = 0.f;
        for (int d = 0; d < V; ++d) s += dO[(hb + g) * V + d] * out[(hb + g) * V + d];
        Dg[g] = s;
        for (int d = 0; d < K; ++d) dq[(hb + g) * K + d] = 0.f;
    }
    for (int l = L - 1; l >= 0; --l) {
        const int Nl = level_n[l];
        const int32_t* par = parents + ((int64_t)l * nq + qi) * TK;
        const int32_t* nxt = l > 0 ? parents + ((int64_t)(l - 1) * nq + qi) * TK : NULL;
        int np = 0; while (np < TK && par[np] >= 0) ++np;
        if (np <= 0) continue;
        int rci = (int)((t / ipow(CR, l)) % CR);
        int nc = (np - 1) * CR + rci + 1, rp = nc - 1;
        const float* cq = cosc + (int64_t)rp * half; const float* sq = sinc + (int64_t)rp * half;
        for (int g = 0; g < G; ++g) {
            rope_fwd(qg + (int64_t)g * K, cq, sq, qr + g * K, K);
            for (int d = 0; d < K; ++d) qr[g * K + d] *= sh->scale;
        }
        memset(dqr, 0, sizeof(float) * G * K);
        int ns = 0; /* walk the (sorted) next-level selection in step with the (ascending) node ids */
        for (int j = 0; j < nc; ++j) {
            int node = par[j / CR] * CR + j % CR;
            if (node < 0 || node >= Nl) { status = -2; continue; }
            if (nxt) {
                while (ns < TK && nxt[ns] >= 0 && nxt[ns] < node) ++ns;
                if (ns < TK && nxt[ns] == node) continue; /* selected: expanded below, not accumulated */
            }
            const float* ck = cosc + (int64_t)j * half; const float* sk = sinc + (int64_t)j * half;
            const float* kn = layers_k[l] + (((int64_t)b * Nl + node) * sh->H_kv + hk) * K;
            const float* vn = layers_v[l] + (((int64_t)b * Nl + node) * sh->H_kv + hk) * V;
            float* dkn = dk_layers[l] + (((int64_t)b * Nl + node) * sh->H_kv + hk) * K;
            float* dvn = dv_layers[l] + (((int64_t)b * Nl + node) * sh->H_kv + hk) * V;
            rope_fwd(kn, ck, sk, kr, K);
            memset(dkr, 0, sizeof(float) * K);
            for (int g = 0; g < G; ++g) {
                float s = 0.f;
                for (int d = 0; d < K; ++d) s += qr[g * K + d] * kr[d];
                float P = expf(s - gmax[hb + g]) / gsum[hb + g];                 /* src/naive.py:379 */
                float dP = 0.f;
                for (int d = 0; d < V; ++d) dP += dO[(hb + g) * V + d] * vn[d];
                float dS = P * (dP - Dg[g]);                                     /* src/naive.py:382 */
                for (int d = 0; d < K; ++d) { dqr[g * K + d] += dS * kr[d]; dkr[d] += dS * qr[g * K + d]; }
                if (atomic) {
                    for (int d = 0; d < V; ++d) {
                        float add = P * dO[(hb + g) * V + d];
                        #pragma omp atomic
                        dvn[d] += add;
                    }
                } else {
                    for (int d = 0; d < V; ++d) dvn[d] += P * dO[(hb + g) * V + d];
                }
            }
            rope_inv(dkr, ck, sk, tmp, K);                                       /* src/naive.py:385 */
            if (atomic) {
                for (int d = 0; d < K; ++d) {
                    #pragma omp atomic
                    dkn[d] += tmp[d];
                }
            } else {
                for (int d = 0; d < K; ++d) dkn[d] += tmp[d];
            }
        }
        for (int g = 0; g < G; ++g) {                                            /* src/naive.py:384 */
            rope_inv(dqr + g * K, cq, sq, tmp, K);
            for (int d = 0; d < K; ++d) dq[(hb + g) * K + d] += sh->scale * tmp[d];
        }
    }
    return status;
}

/*
 * Backward (src/naive.py:333-386), selections taken as constants.
 *   queries NULL: every group of the tensors.  out (AS STORED, i.e. rounded to the input dtype), dO [B,T,H,V];
 *     gmax, gsum [B,T,H]; parents [L,B,T,H_kv,TK]; dq [B,T,H,K].  Parallel over (b,h_kv) units only, serial and in
 *     query order inside a unit, so the float sums are deterministic.
 *   queries [nq,3] (b,t,h_kv): only those groups; out, dO [nq,G,V]; gmax, gsum [nq,G]; parents [L,nq,TK];
 *     dq [nq,G,K].  Parallel over groups with atomic adds into dk/dv (summation order not deterministic); meant for
 *     timing a bounded sample and for checking dq of sampled queries.
 *   dk_layers[l], dv_layers[l]: zero-filled by the caller, accumulated here.  The mean-pool gradient step is
 *   ho_tree_backward_level(), applied by the caller from the top level down.
 */
int ho_backward(const HoShape* sh, const float* q, const float* const* layers_k, const float* const* layers_v,
                const int32_t* level_n, const float* cosc, const float* sinc, const int32_t* queries, int64_t nq_in,
                const float* out, const float* dO, const float* gmax, const float* gsum, const int32_t* parents,
                float* dq, float* const* dk_layers, float* const* dv_layers) {
    const int G = sh->H / sh->H_kv, K = sh->K;
    const int64_t nq = queries ? nq_in : (int64_t)sh->B * sh->T * sh->H_kv;
    int status = 0;
    #pragma omp parallel
    {
        float* qr = (float*)malloc(sizeof(float) * G * K);
        float* kr = (float*)malloc(sizeof(float) * K);
        float* dqr = (float*)malloc(sizeof(float) * G * K);
        float* dkr = (float*)malloc(sizeof(float) * K);
        float* tmp = (float*)malloc(sizeof(float) * K);
        float* Dg = (float*)malloc(sizeof(float) * G);
        if (queries) {
            #pragma omp for schedule(dynamic, 4)
            for (int64_t qi = 0; qi < nq; ++qi) {
                int rc = backward_group(sh, q, layers_k, layers_v, level_n, cosc, sinc, out, dO, gmax, gsum, parents, nq,
                                        qi, queries[3 * qi], queries[3 * qi + 1], queries[3 * qi + 2], dq, dk_layers,
                                        dv_layers, 1, qr, kr, dqr, dkr, tmp, Dg);
                if (rc) status = rc;
            }
        } else {
            #pragma omp for collapse(2) schedule(dynamic, 1)
            for (int b = 0; b < sh->B; ++b)
                for (int hk = 0; hk < sh->H_kv; ++hk)
                    for (int t = 0; t < sh->T; ++t) {
                        int64_t qi = ((int64_t)b * sh->T + t) * sh->H_kv + hk;
                        int rc = backward_group(sh, q, layers_k, layers_v, level_n, cosc, sinc, out, dO, gmax, gsum,
                                                parents, nq, qi, b, t, hk, dq, dk_layers, dv_layers, 0, qr, kr, dqr,
                                                dkr, tmp, Dg);
                        if (rc) status = rc;
                    }
        }
        free(qr); free(kr); free(dqr); free(dkr); free(tmp); free(Dg);
    }
    return status;
}

/* Use n OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1). */
void ho_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int ho_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
