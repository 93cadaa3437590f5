/*
 * sampler_oracle.c -- CPU restatement of the reference sampler.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker, never the product: only tests, the smoke check and the
 * CPU-baseline / reference legs of the benchmark may link or call it.
 *
 * What it restates (citations are into the reference project's files):
 *   - the three CUDA kernels of sampling.cu: top-p only (sampling.cu:757-964), temperature /
 *     top-k / top-p (sampling.cu:517-752) and the repetition-penalty variant (sampling.cu:172-438);
 *   - their block primitives: butterfly all-reduce (sampling.cu:11-46), monotone sequential
 *     combine (sampling.cu:34-42), descending-offset inclusive scan (sampling.cu:48-104),
 *     the Inf/NaN sanitiser sf (sampling.cu:131-134);
 *   - the host-side argument checks and remaps (sampling.cu:451-486, :975-1011);
 *   - the per-row RNG state (sampling.cu:9, :136-144).  The generator itself lives in a
 *     third-party dependency that is not part of the reference tree: cuRAND's device API
 *     (CUDA toolkit 12.9, curandStatePhilox4_32_10_t).  Its published algorithm is
 *     Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
 *     SC'11); it is restated here from the paper, with the documented cuRAND conventions:
 *     key = seed (lo, hi), 128-bit counter, the subsequence added into the counter's high
 *     64 bits, uniform = u32 * 2^-32 + 2^-33 in fp32.
 *
 * Arithmetic model.  The kernels run 1024 threads per row; thread t owns the float4 groups
 * t, t+1024, t+2048, ... of the row.  Every fp32 sum below is carried out with the same
 * association as the CUDA code (per-thread sequential chain, 32-lane tree, 32 warp partials
 * combined by a tree or sequentially), using IEEE fp32 add/mul/div/fma, so that -- GIVEN the
 * same fp32 probabilities -- threshold, compensation factor, lane pick and sampled id are
 * bit-identical to the CUDA kernel.  The one operation that cannot be reproduced on a CPU is
 * exp2f: the GPU evaluates it with a hardware approximation (<= 2 ulp), this file with libm.
 * rs_oracle_sample_row() therefore accepts the probabilities from outside (probs_in) for
 * bit-level checks, and computes its own otherwise.
 *
 * PARITY STATUS: the reference ships no tests, golden vectors or CPU code.  This restatement
 * is pinned (a) for the RNG by the published Philox4x32-10 known-answer vectors and (b) for
 * everything else against the reference's own CUDA extension, compiled unmodified from its
 * sources (oracle/build_ref.py -> oracle/_ref/) and run on the GPU box by the `gpu` tests;
 * fixtures produced that way are committed under tests/golden/.
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -ffp-contract=off -fno-fast-math sampler_oracle.c -lm
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RS_LANES 1024
#define RS_WARPS 32

/* ---------------------------------------------------------------- RNG ------------------ */

typedef struct {
    uint32_t ctr[4];
    uint32_t out[4];
    uint32_t key[2];
    uint32_t pos;          /* cuRAND's STATE: index of the next unused word of out[] */
    int32_t bm_flag;
    int32_t bm_flag_double;
    float bm_extra;
    double bm_extra_double;
} rs_rng_state;            /* 64 bytes, field order of curandStatePhilox4_32_10 */

void rs_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* sampling.cu:136-144: state b <- init(seed, subsequence = row index, offset 0). row0 lets a
 * shard of a larger batch start at its global row index. */
void rs_oracle_setup_rand(uint8_t* states, uint64_t seed, int64_t B, int64_t row0) {
    for (int64_t b = 0; b < B; b++) {
        rs_rng_state st;
        memset(&st, 0, sizeof st);
        uint64_t sub = (uint64_t)(row0 + b);
        st.ctr[2] = (uint32_t)sub;
        st.ctr[3] = (uint32_t)(sub >> 32);
        st.key[0] = (uint32_t)seed;
        st.key[1] = (uint32_t)(seed >> 32);
        rs_oracle_philox4x32_10(st.ctr, st.key, st.out);
        memcpy(states + 64 * b, &st, 64);
    }
}

/* One 4-word draw with cuRAND's curand4 convention: hand out the cached block, bump the
 * counter, refill the cache (sampling.cu:383 draws exactly one such block per call). */
void rs_oracle_draw4(uint8_t* state_bytes, uint32_t r[4]) {
    rs_rng_state st;
    memcpy(&st, state_bytes, 64);
    uint32_t old[4] = {st.out[0], st.out[1], st.out[2], st.out[3]};
    for (int i = 0; i < 4; i++) {
        if (++st.ctr[i] != 0) break;
    }
    rs_oracle_philox4x32_10(st.ctr, st.key, st.out);
    uint32_t s = st.pos & 3u;
    for (int i = 0; i < 4; i++) {
        uint32_t j = s + (uint32_t)i;
        r[i] = (j < 4) ? old[j] : st.out[j - 4];
    }
    memcpy(state_bytes, &st, 64);
}

float rs_oracle_uniform(uint32_t x) {
    const float inv = 2.3283064365386963e-10f; /* 2^-32 */
    return (float)x * inv + (inv / 2.0f);
}

/* ------------------------------------------------------- block primitives -------------- */

static inline float sf(float x) {
    float y = isnan(x) ? 0.0f : x;
    return isinf(y) ? copysignf(FLT_MAX, y) : y;
}

/* 32-lane xor butterfly, offsets 16,8,4,2,1 (sampling.cu:11-17); all lanes end equal. */
static float tree32_f(const float* v) {
    float a[32], b[32];
    memcpy(a, v, sizeof a);
    for (int off = 16; off > 0; off >>= 1) {
        for (int i = 0; i < 32; i++) b[i] = a[i] + a[i ^ off];
        memcpy(a, b, sizeof a);
    }
    return a[31];
}

/* blockReduceAll<Sum>, default flavour: tree per warp, then a tree over the 32 warp values. */
static float block_sum_tree(const float* lane) {
    float w[32];
    for (int i = 0; i < RS_WARPS; i++) w[i] = tree32_f(lane + 32 * i);
    return tree32_f(w);
}

/* blockReduceAll<Sum, monotone_sum=true>: tree per warp, then thread 0 adds w0..w31 in order. */
static float block_sum_seq(const float* lane) {
    float s = tree32_f(lane);
    for (int i = 1; i < RS_WARPS; i++) s += tree32_f(lane + 32 * i);
    return s;
}

/* blockInclusiveScan (sampling.cu:61-104): descending-offset Hillis-Steele per warp, sequential
 * prefix over the warp totals, each lane adds the previous warp's prefix. Returns the total. */
static float block_scan(const float* in, float* out) {
    float wsum[32];
    for (int w = 0; w < RS_WARPS; w++) {
        float a[32], b[32];
        memcpy(a, in + 32 * w, sizeof a);
        for (int off = 16; off > 0; off >>= 1) {
            for (int i = 0; i < 32; i++) b[i] = (i >= off) ? a[i] + a[i - off] : a[i];
            memcpy(a, b, sizeof a);
        }
        memcpy(out + 32 * w, a, sizeof a);
        wsum[w] = a[31];
    }
    float s = wsum[0];
    for (int w = 1; w < RS_WARPS; w++) {
        s += wsum[w];
        wsum[w] = s;
    }
    for (int w = 1; w < RS_WARPS; w++)
        for (int i = 0; i < 32; i++) out[32 * w + i] += wsum[w - 1];
    return out[RS_LANES - 1];
}

/* ------------------------------------------------------------- one row ----------------- */

typedef struct {
    float maxu, denom, pmin, pmax, threshold, comp, sgtp, sum_p, randp, sum_o, rand2;
    uint32_t left, seqk, sgtk, rounds, idxt, early_exit, rnd[4];
    int32_t token;
} rs_oracle_trace;

enum { RS_KIND_TOPP = 0, RS_KIND_GENERAL = 1, RS_KIND_REPETITION = 2 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/*
 * kind 0: batch_sampling_topp_kernel (mass only, scale (float)log2(e));
 * kind 1: batch_sampling_temperature_topk_topp_kernel; kind 2: the repetition kernel.
 * probs_in  (optional, V floats): use these fp32 probabilities instead of computing them.
 * probs_out (optional, V floats): receives the probabilities the search ran on.
 * Returns the sampled id; penalties (kind 2) and the RNG state are updated in place.
 */
int32_t rs_oracle_sample_row(const float* logits, float* penalties, uint8_t* state, int V, int kind, float scale,
                             int top_k, float top_p, float presence, float repetition, float decay,
                             const float* probs_in, float* probs_out, rs_oracle_trace* tr) {
    const int V4 = V / 4;
    float* probs = (float*)malloc(sizeof(float) * (size_t)V);
    float lane[RS_LANES], lane2[RS_LANES], lane3[RS_LANES], cum[RS_LANES];
    uint32_t ulane[RS_LANES];
    rs_oracle_trace T;
    memset(&T, 0, sizeof T);

    if (probs_in) {
        memcpy(probs, probs_in, sizeof(float) * (size_t)V);
        float pmax = -INFINITY, pmin = INFINITY;
        for (int i = 0; i < V; i++) {
            pmax = fmaxf(pmax, probs[i]);
            pmin = fminf(pmin, probs[i]);
        }
        T.pmax = pmax;
        T.pmin = pmin;
    } else {
        /* pass 1 (sampling.cu:208-227 / :547-559 / :784-796): scale, sanitise, row max */
        float maxu = -INFINITY;
        for (int i = 0; i < V; i++) {
            float x;
            if (kind == RS_KIND_REPETITION) x = sf((sf(logits[i]) - penalties[i]) * scale);
            else x = sf(logits[i] * scale);
            probs[i] = x;
            maxu = fmaxf(maxu, x);
        }
        T.maxu = maxu;
        /* pass 2 (sampling.cu:560-572): per-thread chain of 4-sums, tree, tree */
        for (int t = 0; t < RS_LANES; t++) {
            float acc = 0.f;
            for (int i = t; i < V4; i += RS_LANES) {
                float em = 0.f;
                for (int j = 0; j < 4; j++) em += exp2f(probs[4 * i + j] - maxu);
                acc += em;
            }
            lane[t] = acc;
        }
        float denom = block_sum_tree(lane);
        T.denom = denom;
        /* pass 3 (sampling.cu:573-590) */
        float pmax = -INFINITY, pmin = INFINITY;
        for (int i = 0; i < V; i++) {
            float p = exp2f(probs[i] - maxu) / denom;
            probs[i] = p;
            pmax = fmaxf(pmax, p);
            pmin = fminf(pmin, p);
        }
        T.pmax = pmax;
        T.pmin = pmin;
    }
    if (probs_out) memcpy(probs_out, probs, sizeof(float) * (size_t)V);

    /* search (sampling.cu:593-654, :829-878) */
    uint32_t left = f2u(T.pmin), right = f2u(T.pmax) + 1u;
    uint32_t cnt_x = (uint32_t)V;
    float mass_x = 1.0f;
    const int use_cnt = (kind != RS_KIND_TOPP);
    uint32_t rounds = 0;
    for (;;) {
        int go = use_cnt ? (cnt_x > (uint32_t)top_k || mass_x > top_p) : (mass_x > top_p);
        if (!(go && left < right - 1u)) {
            T.early_exit = (left < right - 1u);
            break;
        }
        rounds++;
        uint32_t piv[3];
        piv[1] = (left + right) / 2u;
        piv[0] = (left + piv[1]) / 2u;
        piv[2] = (piv[1] + right) / 2u;
        uint32_t cnt[3];
        float mass[3];
        for (int q = 0; q < 3; q++) {
            const float pv = u2f(piv[q]);
            uint32_t c = 0;
            for (int t = 0; t < RS_LANES; t++) {
                float acc = 0.f;
                for (int i = t; i < V4; i += RS_LANES)
                    for (int j = 0; j < 4; j++) {
                        float p = probs[4 * i + j];
                        if (p >= pv) { c++; acc += p; }
                    }
                lane[t] = acc;
            }
            cnt[q] = c;
            mass[q] = block_sum_seq(lane);
        }
        int ok0 = (use_cnt ? cnt[0] < (uint32_t)top_k : 1) && mass[0] < top_p;
        int ok1 = (use_cnt ? cnt[1] < (uint32_t)top_k : 1) && mass[1] < top_p;
        int ok2 = (use_cnt ? cnt[2] < (uint32_t)top_k : 1) && mass[2] < top_p;
        if (ok0) { right = piv[0]; continue; }
        if (ok1) { left = piv[0]; right = piv[1]; cnt_x = cnt[0]; mass_x = mass[0]; continue; }
        if (ok2) { left = piv[1]; right = piv[2]; cnt_x = cnt[1]; mass_x = mass[1]; continue; }
        left = piv[2]; cnt_x = cnt[2]; mass_x = mass[2];
    }
    T.left = left;
    T.rounds = rounds;
    const float thr = u2f(left);
    T.threshold = thr;

    /* recount (sampling.cu:657-680): per-thread eq / gt counts and gt mass; totals by scan order */
    uint32_t seqk = 0, sgtk = 0;
    for (int t = 0; t < RS_LANES; t++) {
        float gtp = 0.f;
        uint32_t eqk = 0, gtk = 0;
        for (int i = t; i < V4; i += RS_LANES)
            for (int j = 0; j < 4; j++) {
                float p = probs[4 * i + j];
                if (p == thr) eqk++;
                if (p > thr) { gtk++; gtp += p; }
            }
        lane[t] = gtp;
        ulane[t] = eqk;
        seqk += eqk;
        sgtk += gtk;
    }
    float sgtp = block_scan(lane, cum);
    T.sgtp = sgtp; T.seqk = seqk; T.sgtk = sgtk;

    /* compensation (sampling.cu:690-696, :903-908) */
    float comp = 1.0f;
    if (seqk > 0) {
        comp = fminf(sf((top_p - sgtp) / (thr * (float)seqk)), comp);
        if (use_cnt) comp = fminf(sf((float)((uint32_t)top_k - sgtk) / (float)seqk), comp);
        comp = fmaxf(comp, 0.0f);
    }
    T.comp = comp;

    /* lane pick (sampling.cu:699-723). nvcc contracts the last multiply-add into an fma. */
    for (int t = 0; t < RS_LANES; t++) lane2[t] = fmaf(thr * (float)ulane[t], comp, lane[t]);
    float sum_p = block_scan(lane2, cum);
    uint32_t r4[4];
    rs_oracle_draw4(state, r4);
    memcpy(T.rnd, r4, sizeof r4);
    float randp = sum_p * rs_oracle_uniform(r4[0]);
    int idxt = 0;
    {
        int prev = 0;
        for (int t = 0; t < RS_LANES; t++) {
            int u = (randp <= cum[t]);
            if (u != prev) idxt = t; /* monotone scan: at most one transition */
            prev = u;
        }
    }
    T.sum_p = sum_p; T.randp = randp; T.idxt = (uint32_t)idxt;

    /* element pick (sampling.cu:725-751) */
    for (int t = 0; t < RS_LANES; t++) {
        int idn = idxt * 4 + (t / 4) * 4 * RS_LANES + (t % 4);
        float o0 = (idn < V) ? probs[idn] : 0.f;
        lane3[t] = (o0 < thr) ? 0.f : (o0 == thr) ? (o0 * comp) : o0;
    }
    float sum_o = block_scan(lane3, cum);
    float rand2 = sum_o * rs_oracle_uniform(r4[1]);
    int32_t token = 0;
    {
        int prev = 0;
        for (int t = 0; t < RS_LANES; t++) {
            int u = (rand2 <= cum[t]);
            if (u != prev) {
                int idn = idxt * 4 + (t / 4) * 4 * RS_LANES + (t % 4);
                token = (idn < V) ? idn : 0;
            }
            prev = u;
        }
    }
    T.sum_o = sum_o; T.rand2 = rand2; T.token = token;

    /* penalty decay + hit (sampling.cu:427-437) */
    if (kind == RS_KIND_REPETITION) {
        for (int i = 0; i < V; i++) {
            float p = penalties[i];
            penalties[i] = fmaf(p, decay, (i != token) ? 0.f : (p == 0.f ? presence : repetition));
        }
    }
    if (tr) *tr = T;
    free(probs);
    return token;
}

/* ------------------------------------------------- host wrapper semantics -------------- */

/* Argument checks and remaps of the two host functions (sampling.cu:451-486, :975-1011).
 * Returns 0, or a negative code for the conditions on which the reference throws
 * std::invalid_argument: -1 bad V, -2 bad B/T, -3 temperature out of range. */
int rs_oracle_normalise(int64_t V, int64_t B, int64_t T, double temperature, int64_t top_k, double top_p,
                        int with_penalties, int* kind, float* scale, int* top_k_out, float* top_p_out) {
    if (!(V > 0 && V <= 1048576 && V % 4 == 0)) return -1;
    if (!(B > 0 && T > 0)) return -2;
    if (!(temperature >= 0.001 && temperature <= 1000)) return -3;
    if (top_k <= 0 || top_k > V) top_k = V;
    if (top_p < 0 || top_p > 1) top_p = 1;
    if (top_p == 0) { top_k = 1; top_p = 1; }
    double l2 = 1.4426950408889634074 / temperature; /* M_LOG2E / temperature, in double */
    if (with_penalties) *kind = RS_KIND_REPETITION;
    else *kind = (temperature == 1 && top_k == V) ? RS_KIND_TOPP : RS_KIND_GENERAL;
    *scale = (*kind == RS_KIND_TOPP) ? (float)1.4426950408889634074 : (float)l2;
    *top_k_out = (int)top_k;
    *top_p_out = (float)top_p;
    return 0;
}

/* Whole call: rows are independent (one CUDA block per row, sampling.cu:188), so they are
 * spread over the host cores.  logits is (B, T, V) and only position T-1 is read
 * (sampling.cu:202); penalties is (B, V) or NULL; states is B x 64 bytes; out is int32[B]. */
int rs_oracle_sample(const float* logits, float* penalties, uint8_t* states, int32_t* out, int64_t B, int64_t T,
                     int64_t V, double temperature, int64_t top_k, double top_p, double presence, double repetition,
                     double decay, int nthreads) {
    int kind, k;
    float scale, p;
    int rc = rs_oracle_normalise(V, B, T, temperature, top_k, top_p, penalties != NULL, &kind, &scale, &k, &p);
    if (rc) return rc;
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
    for (int64_t b = 0; b < B; b++) {
        const float* row = logits + (b * T + (T - 1)) * V;
        float* pen = penalties ? penalties + b * V : NULL;
        out[b] = rs_oracle_sample_row(row, pen, states + 64 * b, (int)V, kind, scale, k, p, (float)presence,
                                      (float)repetition, (float)decay, NULL, NULL, NULL);
    }
    return 0;
}

/* ------------------------------------------------------ exported primitives (tests) ---- */

/* The 1024-wide inclusive scan used for the lane / element picks. Returns the total. */
float rs_oracle_block_scan(const float* in, float* out) { return block_scan(in, out); }

/* The variant the reference rejects (sampling.cu:79-83 and monotonicity.py): ascending offsets.
 * Kept only so that a test can show it is NOT monotone while the descending one is. */
void rs_oracle_warp_scan_ascending(const float* in, float* out, int n) {
    float* a = (float*)malloc(sizeof(float) * (size_t)n);
    float* b = (float*)malloc(sizeof(float) * (size_t)n);
    memcpy(a, in, sizeof(float) * (size_t)n);
    for (int off = 1; off < n; off <<= 1) {
        for (int i = 0; i < n; i++) b[i] = (i >= off) ? a[i] + a[i - off] : a[i];
        memcpy(a, b, sizeof(float) * (size_t)n);
    }
    memcpy(out, a, sizeof(float) * (size_t)n);
    free(a);
    free(b);
}

/* Descending offsets over n (a power of two) values: the order of sampling.cu:48-58 generalised. */
void rs_oracle_warp_scan_descending(const float* in, float* out, int n) {
    float* a = (float*)malloc(sizeof(float) * (size_t)n);
    float* b = (float*)malloc(sizeof(float) * (size_t)n);
    memcpy(a, in, sizeof(float) * (size_t)n);
    for (int off = n / 2; off > 0; off >>= 1) {
        for (int i = 0; i < n; i++) b[i] = (i >= off) ? a[i] + a[i - off] : a[i];
        memcpy(a, b, sizeof(float) * (size_t)n);
    }
    memcpy(out, a, sizeof(float) * (size_t)n);
    free(a);
    free(b);
}

float rs_oracle_block_sum_tree(const float* lane) { return block_sum_tree(lane); }
float rs_oracle_block_sum_seq(const float* lane) { return block_sum_seq(lane); }
float rs_oracle_sf(float x) { return sf(x); }
