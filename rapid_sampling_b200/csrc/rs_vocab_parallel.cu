// Vocab-parallel sampling: each GPU holds V/N columns of every row (what a tensor-parallel lm_head
// produces).  No reference counterpart -- the reference is single-GPU only (sampling.cu has no
// collective anywhere); the semantics are those of its kernels (softmax of penalised, scaled logits;
// kept set {p >= v}; fractional weight for ties with v, sampling.cu:365-371, :690-696), evaluated on the
// union of the shards.
//
// The work is cut into small per-shard kernels with a collective between them (issued by the host
// driver over NCCL):
//   vp_max      row maximum of the sanitised scaled logits of this shard           -> all-reduce MAX
//   vp_sum      sum of exp2(x - max) over this shard                                -> all-reduce SUM
//   vp_round    counts and masses of this shard at 15 pivots between (left, right)  -> all-reduce SUM
//               (8 rounds of a 16-ary search over the fp32 bit patterns of p; every rank derives the
//                same new bracket from the same reduced numbers, so no decision is ever exchanged)
//   vp_tally    at the threshold: count above, mass above, ties                     -> all-reduce SUM
//   vp_weight   this shard's kept weight                                            -> all-gather
//   vp_pick     the owner shard (first whose prefix reaches u * total) picks the id -> all-reduce MAX
// Sums inside a shard are fp32 in a fixed order (per-thread chain, warp tree, warp values in order), so a
// run is deterministic; across shards NCCL delivers identical bits to every rank.  Results are not
// bit-identical to the single-GPU kernel (its per-lane chains are cut at shard borders); they obey the
// same float64 kept-set and chi-square checks.
#include "rs_device.cuh"
#include "../../include/rapid_sampling_b200.h"

namespace rs {

constexpr int kVpThreads = 1024;
constexpr int kVpPivots = 15;

struct VpRow {
    const float* logits;   // this shard's columns of the row (position T-1)
    float* penalties;      // this shard's columns or null
    int n;                 // columns in this shard
};

__device__ __forceinline__ VpRow vp_row(const float* logits, long long row_stride, float* penalties, int n, int b) {
    VpRow r;
    r.logits = logits + (long long)b * row_stride;
    r.penalties = penalties ? penalties + (long long)b * n : nullptr;
    r.n = n;
    return r;
}
__device__ __forceinline__ float vp_x(const VpRow& r, int i, float scale) {
    const float l = r.logits[i];
    return r.penalties ? sanitize((sanitize(l) - r.penalties[i]) * scale) : sanitize(l * scale);
}

// block-wide fixed-order sum: per-thread value -> warp tree -> 32 warp values added in order by every thread
__device__ __forceinline__ float vp_block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = warp_tree_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float s = sh[0];
#pragma unroll
    for (int i = 1; i < kVpThreads / 32; i++) s += sh[i];
    return s;
}

__global__ void __launch_bounds__(kVpThreads) vp_max_kernel(const float* logits, long long row_stride, float* penalties,
                                                            int n, float scale, float* out_max) {
    __shared__ float sh[32];
    const VpRow r = vp_row(logits, row_stride, penalties, n, blockIdx.x);
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += kVpThreads) m = fmaxf(m, vp_x(r, i, scale));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = warp_max(sh[threadIdx.x]);
        if (threadIdx.x == 0) out_max[blockIdx.x] = m;
    }
}

__global__ void __launch_bounds__(kVpThreads) vp_sum_kernel(const float* logits, long long row_stride, float* penalties,
                                                            int n, float scale, const float* gmax, float* out_sum) {
    __shared__ float sh[32];
    const VpRow r = vp_row(logits, row_stride, penalties, n, blockIdx.x);
    const float mx = gmax[blockIdx.x];
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += kVpThreads) acc += exp2f(vp_x(r, i, scale) - mx);
    const float s = vp_block_sum(acc, sh);
    if (threadIdx.x == 0) out_sum[blockIdx.x] = s;
}

// Bracket update shared by every kernel that needs the current (left, right): the bracket after `rounds_done`
// rounds is recomputed from the reduced tallies of all rounds so far -- pure integer / compare logic on numbers
// that are identical on every rank.
struct VpBracket { uint32_t left, right; };
__device__ __forceinline__ void vp_pivots(uint32_t left, uint32_t right, uint32_t piv[kVpPivots]) {
    const unsigned long long w = (unsigned long long)(right - left);
#pragma unroll
    for (int j = 0; j < kVpPivots; j++) piv[j] = left + (uint32_t)((w * (unsigned)(j + 1)) >> 4);
}
__device__ __forceinline__ VpBracket vp_bracket(const float* tallies /* [round][B][15][2] reduced */, int B, int b,
                                                int rounds_done, float top_k, float top_p) {
    VpBracket br;
    br.left = 0u;              // the set {p >= 0} is the whole row: never "fewer than top_k"
    br.right = 0x3f800001u;    // above 1.0f: the empty set
    for (int r = 0; r < rounds_done; r++) {
        if (br.right - br.left <= 1u) break;   // converged: later rounds carry no data
        uint32_t piv[kVpPivots];
        vp_pivots(br.left, br.right, piv);
        const float* t = tallies + (((long long)r * B + b) * kVpPivots) * 2;
        uint32_t nl = br.left, nr = br.right;
        bool found_right = false;
#pragma unroll
        for (int j = 0; j < kVpPivots; j++) {
            const bool ok = (t[2 * j] < top_k) && (t[2 * j + 1] < top_p);   // fewer than top_k AND less than top_p mass
            if (!ok) nl = piv[j];
            else if (!found_right) { nr = piv[j]; found_right = true; }
        }
        br.left = nl;
        br.right = nr;
    }
    return br;
}

// One round: this shard's count and mass at the 15 pivots of the current bracket.
__global__ void __launch_bounds__(kVpThreads) vp_round_kernel(const float* logits, long long row_stride, float* penalties,
                                                              int n, float scale, const float* gmax, const float* gsum,
                                                              const float* tallies, int B, int round, float top_k,
                                                              float top_p, float* out /* [B][15][2] */) {
    __shared__ float sh[32];
    const int b = blockIdx.x;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const float mx = gmax[b], denom = gsum[b];
    const VpBracket br = vp_bracket(tallies, B, b, round, top_k, top_p);
    uint32_t piv[kVpPivots];
    vp_pivots(br.left, br.right, piv);
    float cnt[kVpPivots], mass[kVpPivots];
#pragma unroll
    for (int j = 0; j < kVpPivots; j++) cnt[j] = mass[j] = 0.f;
    if (br.right - br.left > 1u) {
        for (int i = threadIdx.x; i < n; i += kVpThreads) {
            const float p = exp2f(vp_x(r, i, scale) - mx) / denom;
            const uint32_t pb = __float_as_uint(p);
#pragma unroll
            for (int j = 0; j < kVpPivots; j++)
                if (pb >= piv[j]) { cnt[j] += 1.f; mass[j] += p; }
        }
    }
#pragma unroll
    for (int j = 0; j < kVpPivots; j++) {
        const float c = vp_block_sum(cnt[j], sh);
        const float m = vp_block_sum(mass[j], sh);
        if (threadIdx.x == 0) {
            out[((long long)b * kVpPivots + j) * 2] = c;
            out[((long long)b * kVpPivots + j) * 2 + 1] = m;
        }
    }
}

// At the threshold (= left after all rounds): count above, mass above, ties, in this shard.
__global__ void __launch_bounds__(kVpThreads) vp_tally_kernel(const float* logits, long long row_stride, float* penalties,
                                                              int n, float scale, const float* gmax, const float* gsum,
                                                              const float* tallies, int B, int rounds, float top_k,
                                                              float top_p, float* out /* [B][4] */) {
    __shared__ float sh[32];
    const int b = blockIdx.x;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const float mx = gmax[b], denom = gsum[b];
    const uint32_t thr = vp_bracket(tallies, B, b, rounds, top_k, top_p).left;
    float cgt = 0.f, mgt = 0.f, ceq = 0.f;
    for (int i = threadIdx.x; i < n; i += kVpThreads) {
        const float p = exp2f(vp_x(r, i, scale) - mx) / denom;
        const uint32_t pb = __float_as_uint(p);
        if (pb > thr) { cgt += 1.f; mgt += p; }
        if (pb == thr) ceq += 1.f;
    }
    const float a = vp_block_sum(cgt, sh), m = vp_block_sum(mgt, sh), e = vp_block_sum(ceq, sh);
    if (threadIdx.x == 0) {
        out[b * 4] = a; out[b * 4 + 1] = m; out[b * 4 + 2] = e; out[b * 4 + 3] = 0.f;
    }
}

__device__ __forceinline__ float vp_comp(const float* gt /* reduced [4] */, float thr, float top_k, float top_p, bool use_p) {
    float comp = 1.0f;
    const float sgtk = gt[0], sgtp = gt[1], seqk = gt[2];
    if (seqk > 0.f) {
        if (use_p) comp = fminf(sanitize((top_p - sgtp) / (thr * seqk)), comp);
        comp = fminf(sanitize((top_k - sgtk) / seqk), comp);
        comp = fmaxf(comp, 0.0f);
    }
    return comp;
}
__device__ __forceinline__ float vp_weight_of(float p, float thr, float comp) {
    return (p < thr) ? 0.f : (p == thr) ? p * comp : p;
}

// This shard's kept weight, written into column `rank` of a [B][N] matrix that is then summed over ranks.
__global__ void __launch_bounds__(kVpThreads) vp_weight_kernel(const float* logits, long long row_stride, float* penalties,
                                                               int n, float scale, const float* gmax, const float* gsum,
                                                               const float* tallies, int B, int rounds, float top_k,
                                                               float top_p, int use_p, const float* gtally, int rank,
                                                               int world, float* out /* [B][world] */) {
    __shared__ float sh[32];
    const int b = blockIdx.x;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const float mx = gmax[b], denom = gsum[b];
    const float thr = __uint_as_float(vp_bracket(tallies, B, b, rounds, top_k, top_p).left);
    const float comp = vp_comp(gtally + b * 4, thr, top_k, top_p, use_p != 0);
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += kVpThreads)
        acc += vp_weight_of(exp2f(vp_x(r, i, scale) - mx) / denom, thr, comp);
    const float s = vp_block_sum(acc, sh);
    if (threadIdx.x == 0) out[(long long)b * world + rank] = s;
}

// Owner election and pick.  Every rank sees the same [B][N] weights and the same uniform draw, so every rank
// names the same owner; the owner walks its shard in column order (chunks of 1024 columns, block scan) to the
// first kept column whose running weight reaches the target and reports global id + 1; the others report 0.
__global__ void __launch_bounds__(kVpThreads) vp_pick_kernel(const float* logits, long long row_stride, float* penalties,
                                                             int n, float scale, const float* gmax, const float* gsum,
                                                             const float* tallies, int B, int rounds, float top_k,
                                                             float top_p, int use_p, const float* gtally,
                                                             const float* weights /* reduced [B][world] */, int rank,
                                                             int world, unsigned char* states, long long col0,
                                                             int* out_plus1 /* [B] */) {
    __shared__ float sh[32];
    __shared__ float s_run;
    __shared__ int s_found, s_last;
    const int b = blockIdx.x, t = threadIdx.x, lane = t & 31, w = t >> 5;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const float mx = gmax[b], denom = gsum[b];
    const float thr = __uint_as_float(vp_bracket(tallies, B, b, rounds, top_k, top_p).left);
    const float comp = vp_comp(gtally + b * 4, thr, top_k, top_p, use_p != 0);
    RngWords rng;
    {
        const uint4* st = reinterpret_cast<const uint4*>(states + (long long)b * RS_STATE_BYTES);
        rng.ctr = st[0]; rng.block = st[1]; rng.key_pos = st[2];
    }
    uint32_t r0, r1, r4[4];
    rng_peek2(rng, r0, r1, r4);
    float total = 0.f;
    for (int k = 0; k < world; k++) total += weights[(long long)b * world + k];
    const float target = total * u01(r0);
    int owner = -1;
    float before = 0.f, run = 0.f;
    int last_nonzero = 0;
    float before_last = 0.f;
    for (int k = 0; k < world; k++) {
        const float wk = weights[(long long)b * world + k];
        if (wk > 0.f) { last_nonzero = k; before_last = run; }
        const float nxt = run + wk;
        if (owner < 0 && wk > 0.f && target <= nxt) { owner = k; before = run; }
        run = nxt;
    }
    if (owner < 0) { owner = last_nonzero; before = before_last; }   // rounding only
    __syncthreads();
    if (t == 0) {   // every rank advances its replica of the state by one 4-word block
        const uint4 nctr = ctr_next(rng.ctr);
        uint4* st = reinterpret_cast<uint4*>(states + (long long)b * RS_STATE_BYTES);
        st[0] = nctr;
        st[1] = philox4x32_10(nctr, rng.key_pos.x, rng.key_pos.y);
        s_run = before;
        s_found = 0x7fffffff;
        s_last = -1;
    }
    __syncthreads();
    if (rank != owner) {
        if (t == 0) out_plus1[b] = 0;
        return;
    }
    for (int base = 0; base < n; base += kVpThreads) {
        const int i = base + t;
        const float wv = (i < n) ? vp_weight_of(exp2f(vp_x(r, i, scale) - mx) / denom, thr, comp) : 0.f;
        const float incl = warp_scan_desc(wv, lane);
        if (lane == 31) sh[w] = incl;
        __syncthreads();
        float pre = s_run;
        for (int k = 0; k < w; k++) pre += sh[k];
        if (wv > 0.f) {
            atomicMax(&s_last, i);
            if (target <= pre + incl) atomicMin(&s_found, i);
        }
        __syncthreads();
        if (s_found != 0x7fffffff) break;
        if (t == 0) {
            float tot = s_run;
            for (int k = 0; k < 32; k++) tot += sh[k];
            s_run = tot;
        }
        __syncthreads();
    }
    if (t == 0) {
        const int idx = (s_found != 0x7fffffff) ? s_found : max(s_last, 0);
        out_plus1[b] = (int)(col0 + idx) + 1;
    }
}

// Penalty update of this shard's columns (sampling.cu:427-437): decay everything, add the hit on the sampled id.
__global__ void vp_penalty_kernel(float* penalties, int n, int B, const int* ids_plus1 /* reduced */, long long col0,
                                  float presence, float repetition, float decay, const int* gate) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * n) return;
    if (gate && *gate == 0) return;   // fast protocol: some row could not be settled, the call is repeated as a whole
    const int b = (int)(i / n), c = (int)(i - (long long)b * n);
    const float old = penalties[i];
    const bool hit = (col0 + c) == (long long)(ids_plus1[b] - 1);
    penalties[i] = fmaf(old, decay, hit ? (old == 0.f ? presence : repetition) : 0.f);
}

// workspace layout in floats
struct VpLayout { size_t gmax, gsum, tallies, gtally, weights, ids, total; };
static VpLayout vp_layout(long long B, int world) {
    VpLayout l;
    size_t o = 0;
    auto take = [&](size_t n) { size_t at = o; o += (n + 63) & ~(size_t)63; return at; };
    l.gmax = take(B);
    l.gsum = take(B);
    l.tallies = take((size_t)RS_VP_ROUNDS * B * kVpPivots * 2);
    l.gtally = take((size_t)B * 4);
    l.weights = take((size_t)B * world);
    l.ids = take(B);
    l.total = o;
    return l;
}


// =====================================================================================================
// Fast protocol: 3 collectives.  Each shard extracts a short candidate list (every element whose
// e = exp2(x - max) reaches a bound), the lists are all-gathered, and every rank finishes the row
// redundantly on the union -- cutoff search, tie weight, owner-free pick -- from identical data, so the id
// needs no exchange.  The bound is read off a histogram of e by octave that travels with the denominator:
// the largest power of two above which the row still holds more than top_k + 1 elements, or more than top_p
// of the mass; no such octave means "take everything", which only fits short rows.  A row whose candidates
// cannot settle the cutoff (too little mass or too few elements above the bound, or a list overflow) is
// flagged; the driver then repeats the call with the staged protocol above.
//   vpf_max     per (row, sub-block): max of x                                  -> all-reduce MAX  [B][S]
//   vpf_sum     per (row, sub-block): denominator partial, octave histogram     -> all-reduce SUM  [B][S][2 + 2*32]
//               (count and mass per octave; exact in the top 10 octaves, a 1-in-64 sample of groups below)
//   vpf_extract per (row, sub-block): ordered list of (e, column) with e >= bound,
//               written into the sub-block's segment of the row's list           -> all-gather  [B][S][Lmax/S][2] + counts
//   vpf_finish  per row, on every rank: probabilities staged in shared memory, threshold, weights, pick; validity
// =====================================================================================================
constexpr int kFCap = 12;       // candidates a thread may hold per sub-block (96 KiB of shared memory: two CTAs per SM)
constexpr int kFMaxSub = 8;
constexpr int kFBins = 32;      // octaves of e = exp2(x - max) below 1 that the mass histogram resolves
// candidates a rank may contribute per row: the union over ranks stays near 32K entries
__host__ __device__ constexpr int f_lmax(int world) { return (32768 / world) < 2048 ? 2048 : (32768 / world); }

struct FSub { int g0, g1; };    // float4 groups [g0, g1) of the shard handled by a sub-block
__device__ __forceinline__ FSub f_sub(int n, int S, int s) {
    const int G = n >> 2, per = (G + S - 1) / S;
    FSub r;
    r.g0 = min(s * per, G);
    r.g1 = min(r.g0 + per, G);
    return r;
}
// The shard passes are latency-bound when a thread has one load in flight: they fetch kFAhead groups ahead of the
// arithmetic (raw logits and penalties first, the scaling afterwards, in the same order as before).
constexpr int kFAhead = 2;
struct FRaw { float4 l, q; };
__device__ __forceinline__ FRaw vp_raw4(const VpRow& r, int g) {
    FRaw x;
    x.l = reinterpret_cast<const float4*>(r.logits)[g];
    x.q = r.penalties ? reinterpret_cast<const float4*>(r.penalties)[g] : make_float4(0.f, 0.f, 0.f, 0.f);
    return x;
}
__device__ __forceinline__ float4 vp_x4_of(const VpRow& r, const FRaw& x, float scale) {
    float4 v = x.l;
    if (r.penalties) {
        const float4 q = x.q;
        v.x = sanitize((sanitize(v.x) - q.x) * scale); v.y = sanitize((sanitize(v.y) - q.y) * scale);
        v.z = sanitize((sanitize(v.z) - q.z) * scale); v.w = sanitize((sanitize(v.w) - q.w) * scale);
    } else {
        v.x = sanitize(v.x * scale); v.y = sanitize(v.y * scale); v.z = sanitize(v.z * scale); v.w = sanitize(v.w * scale);
    }
    return v;
}
// calls body(g, x4) for this thread's groups g0 + t, g0 + t + 1024, ... < g1, in that order
template <class F>
__device__ __forceinline__ void vp_for_groups(const VpRow& r, int g0, int g1, float scale, F&& body) {
    for (int g = g0 + (int)threadIdx.x; g < g1; g += kFAhead * kVpThreads) {
        FRaw raw[kFAhead];
#pragma unroll
        for (int u = 0; u < kFAhead; u++)
            if (g + u * kVpThreads < g1) raw[u] = vp_raw4(r, g + u * kVpThreads);
#pragma unroll
        for (int u = 0; u < kFAhead; u++)
            if (g + u * kVpThreads < g1) body(g + u * kVpThreads, vp_x4_of(r, raw[u], scale));
    }
}
__device__ __forceinline__ float4 vp_x4(const VpRow& r, int g, float scale) {
    float4 v = reinterpret_cast<const float4*>(r.logits)[g];
    if (r.penalties) {
        const float4 q = reinterpret_cast<const float4*>(r.penalties)[g];
        v.x = sanitize((sanitize(v.x) - q.x) * scale); v.y = sanitize((sanitize(v.y) - q.y) * scale);
        v.z = sanitize((sanitize(v.z) - q.z) * scale); v.w = sanitize((sanitize(v.w) - q.w) * scale);
    } else {
        v.x = sanitize(v.x * scale); v.y = sanitize(v.y * scale); v.z = sanitize(v.z * scale); v.w = sanitize(v.w * scale);
    }
    return v;
}

__global__ void __launch_bounds__(kVpThreads) vpf_max_kernel(const float* logits, long long row_stride, float* penalties, int n,
                                                             float scale, int S, float* stat1, int* all_valid) {
    __shared__ float sh[32];
    const int b = blockIdx.x / S, s = blockIdx.x % S, t = threadIdx.x, lane = t & 31, w = t >> 5;
    if (blockIdx.x == 0 && t == 0) *all_valid = 1;   // cleared by the finishing kernel of any row that cannot be settled
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const FSub sb = f_sub(n, S, s);
    float tmax = -INFINITY;
    for (int g = sb.g0 + t; g < sb.g1; g += kVpThreads) {
        const float4 v = vp_x4(r, g, scale);
        tmax = fmaxf(fmaxf(tmax, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    const float wmax = warp_max(tmax);
    if (lane == 0) sh[w] = wmax;
    __syncthreads();
    if (t < 32) {
        const float mx = warp_max(sh[t]);
        if (t == 0) stat1[b * S + s] = mx;
    }
}

// lm_head epilogue hook, first stage fed tile by tile.  A producer of logits (the epilogue of a tensor-parallel lm_head
// GEMM, or this kernel run on a tile it has just written) folds a tile's row maxima into stat1 as the tile appears, so
// that no separate pass over the shard is needed for the maximum.  The fold is an atomic maximum, hence independent of
// the order in which tiles arrive.  Only slot 0 of a row's S sub-block slots is used; the others stay at -inf.
__device__ __forceinline__ void vp_fold_row_max(float* slot, float v) {
    if (v >= 0.f) atomicMax(reinterpret_cast<int*>(slot), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int*>(slot), __float_as_uint(v));
}
__global__ void vpf_tile_begin_kernel(float* stat1, int n, int* all_valid) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stat1[i] = -INFINITY;
    if (i == 0) *all_valid = 1;
}
// one CTA per (row, chunk of 4096 columns of the tile); ld = elements between consecutive rows of the tile buffer
__global__ void __launch_bounds__(256) vpf_tile_max_kernel(const float* tile, long long ld, const float* pen_tile, long long pen_ld,
                                                           int ncols, float scale, int S, float* stat1) {
    __shared__ float sh[8];
    const int b = blockIdx.y, t = threadIdx.x;
    const float* lrow = tile + (long long)b * ld;
    const float* prow = pen_tile ? pen_tile + (long long)b * pen_ld : nullptr;
    const int c0 = blockIdx.x * 4096, c1 = min(c0 + 4096, ncols);
    float m = -INFINITY;
    for (int c = c0 + t; c < c1; c += 256) {
        const float l = lrow[c];
        const float x = prow ? sanitize((sanitize(l) - prow[c]) * scale) : sanitize(l * scale);
        m = fmaxf(m, x);
    }
    m = warp_max(m);
    if ((t & 31) == 0) sh[t >> 5] = m;
    __syncthreads();
    if (t < 32) {
        m = warp_max(t < 8 ? sh[t] : -INFINITY);
        if (t == 0) vp_fold_row_max(stat1 + (size_t)b * S, m);
    }
}

__device__ __forceinline__ float f_gmax(const float* stat1, int S, int b) {
    float mx = -INFINITY;
    for (int s = 0; s < S; s++) mx = fmaxf(mx, stat1[b * S + s]);
    return mx;
}
// stat2 per (row, sub-block): [0] denominator partial, [1] unused, [2..] histogram: for octave k (e in [2^-(k+1), 2^-k),
// e = 1 counted in octave 0) mass at [2 + 2k] and count at [3 + 2k]
constexpr int kFStat2 = 2 + 2 * kFBins;
__device__ __forceinline__ float f_denom(const float* stat2, int S, int b) {
    float d = 0.f;
    for (int s = 0; s < S; s++) d += stat2[(size_t)(b * S + s) * kFStat2];
    return d;
}
// The candidate bound: the largest power of two 2^-(K+1) such that the octaves 0..K together hold more than top_k
// elements or about top_p of the mass (a forecast from unordered sums; the finishing kernel checks exactly).
// Returns 0 when even all resolved octaves are not enough.
__device__ __forceinline__ float f_bound_e(const float* stat2, int S, int b, float denom, float top_k, float top_p) {
    float cm = 0.f, cc = 0.f;
    for (int k = 0; k < kFBins; k++) {
        for (int s = 0; s < S; s++) {
            cm += stat2[(size_t)(b * S + s) * kFStat2 + 2 + 2 * k];
            cc += stat2[(size_t)(b * S + s) * kFStat2 + 3 + 2 * k];
        }
        if (cc > top_k + 1.f || cm > top_p * denom * 1.001f) return exp2f(-(float)(k + 1));
    }
    return 0.f;
}

// pass 2: denominator partial and the octave histogram of the large elements.  The histogram masses are accumulated
// as integers: an element of octave k is e = m * 2^-(k + 24) with an integer m < 2^24 (its significand), so the sum of
// the m's of up to 2^20 elements fits 64 bits and does not depend on the order in which the atomics land -- the
// bound every rank derives from the reduced histogram is the same in every run.
__global__ void __launch_bounds__(kVpThreads) vpf_sum_kernel(const float* logits, long long row_stride, float* penalties, int n,
                                                             float scale, int S, const float* stat1, float* stat2) {
    __shared__ float sh[32];
    __shared__ unsigned long long hist_m[32][kFBins];   // one histogram per warp: atomics only collide inside a warp
    __shared__ unsigned int hist_c[32][kFBins];
    const int b = blockIdx.x / S, s = blockIdx.x % S, t = threadIdx.x, w = t >> 5;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const FSub sb = f_sub(n, S, s);
    const float gmax = f_gmax(stat1, S, b);
    for (int i = t; i < 32 * kFBins; i += kVpThreads) {
        (&hist_m[0][0])[i] = 0ull;
        (&hist_c[0][0])[i] = 0u;
    }
    __syncthreads();
    float acc = 0.f;
    for (int g = sb.g0 + t; g < sb.g1; g += kVpThreads) {
        const float4 v = vp_x4(r, g, scale);
        const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float d = x[j] - gmax;
            const float e = exp2f(d);
            acc += e;
            // The histogram only steers the choice of the bound (the finishing kernel checks the result exactly), so
            // below the top ten octaves one group in 64 stands for its neighbours: few shared-memory atomics.
            // (one octave of slack in the cheap test; the exact octave decides)
            if (d > -11.f || ((g & 63) == 0 && d > -(float)kFBins)) {
                int k = (int)(-d);                 // octave: e in (2^-(k+1), 2^-k]
                if (e < exp2f(-(float)k) * 0.5f) k++;      // guard the octave edge against rounding of exp2f
                if (k < 10 || (g & 63) == 0) {
                    if (k < kFBins) {
                        atomicAdd(&hist_m[w][k], (unsigned long long)__float2uint_rn(ldexpf(e, k + 24)));
                        atomicAdd(&hist_c[w][k], 1u);
                    }
                }
            }
        }
    }
    const float d = vp_block_sum(acc, sh);
    __syncthreads();
    float* o = stat2 + (size_t)(b * S + s) * kFStat2;
    if (t == 0) { o[0] = d; o[1] = 0.f; }
    if (t < kFBins) {
        unsigned long long m = 0ull;
        unsigned int c = 0u;
        for (int k = 0; k < 32; k++) { m += hist_m[k][t]; c += hist_c[k][t]; }
        const float wgt = (t < 10) ? 1.f : 64.f;       // octaves below the top ten were sampled 1-in-64
        o[2 + 2 * t] = ldexpf((float)m, -(t + 24)) * wgt;
        o[3 + 2 * t] = (float)c * wgt;
    }
}

// pass 3: every element with e >= bound, as (e, global column), in the fixed order (thread, position within the thread),
// written straight into this sub-block's segment of the list that is all-gathered next.  A thread first collects its
// candidates in shared memory (at most kFCap), a block scan of the counts gives every thread its place, and the entries
// are copied in that order; a thread or segment that overflows marks the segment, which makes the finishing kernel
// reject the row (the driver then repeats the call with the staged protocol).
__global__ void __launch_bounds__(kVpThreads) vpf_extract_kernel(const float* logits, long long row_stride, float* penalties,
                                                                 int n, float scale, int S, const float* stat1,
                                                                 const float* stat2, float top_k, float top_p, int seg,
                                                                 uint32_t* send /* [B][S][seg][2] */,
                                                                 uint32_t* send_cnt /* [B][S] */, long long col0) {
    extern __shared__ uint2 s_ent[];       // [kFCap][kVpThreads]
    __shared__ uint32_t s_wsum[32];
    const int b = blockIdx.x / S, s = blockIdx.x % S, t = threadIdx.x, lane = t & 31, w = t >> 5;
    const VpRow r = vp_row(logits, row_stride, penalties, n, b);
    const FSub sb = f_sub(n, S, s);
    const float gmax = f_gmax(stat1, S, b);
    const float denom = f_denom(stat2, S, b);
    const float bound = f_bound_e(stat2, S, b, denom, top_k, top_p);
    uint32_t nc = 0;
    if (bound > 0.f) {
        const float bx = log2f(bound) - 1.f;       // cheap pre-test in the x domain, one octave of slack
        vp_for_groups(r, sb.g0, sb.g1, scale, [&](int g, float4 v) {
            const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (x[j] - gmax >= bx) {
                    const float e = exp2f(x[j] - gmax);
                    if (e >= bound) {
                        if (nc < (uint32_t)kFCap) s_ent[nc * kVpThreads + t] = make_uint2(__float_as_uint(e), (uint32_t)(col0 + 4 * g + j));
                        nc++;
                    }
                }
            }
        });
    } else {
        nc = kFCap + 1;     // no usable bound: flag the row through the overflow path
    }
    const uint32_t c = min(nc, (uint32_t)kFCap);
    uint32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_wsum[w] = incl;
    const int over = __syncthreads_or(nc > (uint32_t)kFCap ? 1 : 0);
    uint32_t pre = 0, tot = 0;
    for (int k = 0; k < 32; k++) {
        const uint32_t x = s_wsum[k];
        pre += (k < w) ? x : 0u;
        tot += x;
    }
    const bool bad = over || tot > (uint32_t)seg;
    if (!bad) {
        uint2* dst = reinterpret_cast<uint2*>(send) + (size_t)(b * S + s) * seg + (pre + incl - c);
        for (uint32_t i = 0; i < c; i++) dst[i] = s_ent[i * kVpThreads + t];
    }
    if (t == 0) send_cnt[b * S + s] = bad ? 0xffffffffu : tot;
}

// block-wide fixed-order sums of NV per-thread values at once: warp trees, then threads 0..NV-1 add the 32 warp values
template <int NV>
__device__ __forceinline__ void f_block_sums(float (&v)[NV], float* sh /* [32][NV] + [NV] */) {
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
#pragma unroll
    for (int i = 0; i < NV; i++) v[i] = warp_tree_sum(v[i]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NV; i++) sh[w * NV + i] = v[i];
    }
    __syncthreads();
    if (t < NV) {
        float a = sh[t];
        for (int k = 1; k < 32; k++) a += sh[k * NV + t];
        sh[32 * NV + t] = a;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; i++) v[i] = sh[32 * NV + i];
}

// The same for 30 values at once (the 15 pivots of a round): the warp stage is a transposing butterfly -- at offset 16 a
// lane keeps 16 of the 32 partial sums and hands the other 16 to its partner, at offset 8 it keeps 8, ... -- 31 shuffles
// instead of 150, after which lane l holds the warp's total of value l.  Fixed order, identical on every rank.
__device__ __forceinline__ void f_block_sums30(float (&v)[30], float* sh /* [32][32] + [32] */) {
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    float a[32];
#pragma unroll
    for (int i = 0; i < 30; i++) a[i] = v[i];
    a[30] = a[31] = 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < o; i++) {
            const float keep = up ? a[i + o] : a[i], give = up ? a[i] : a[i + o];
            a[i] = keep + __shfl_xor_sync(0xffffffffu, give, o);
        }
    }
    __syncthreads();
    sh[w * 32 + lane] = a[0];
    __syncthreads();
    if (t < 32) {
        float x = sh[t];
        for (int k = 1; k < 32; k++) x += sh[k * 32 + t];
        sh[32 * 32 + t] = x;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 30; i++) v[i] = sh[32 * 32 + i];
}

// gath / gath_cnt: the lists and counts of all ranks as ONE all-gather delivered them: rank r's block starts r * rstride
// words on, its lists first ([B][S][seg][2]), its counts ([B][S]) behind them.
__global__ void __launch_bounds__(kVpThreads) vpf_finish_kernel(int B, int S, int world, int seg, const float* stat1, const float* stat2,
                                                                const uint32_t* gath, const uint32_t* gath_cnt, size_t rstride, float top_k,
                                                                float top_p, int use_p, const unsigned char* states,
                                                                int* ids, int* valid) {
    __shared__ float sh[32 * 32 + 32];
    __shared__ float s_scan[32];
    __shared__ int s_hit;
    __shared__ uint32_t s_segoff[kFMaxSub * 8 + 1];   // first flat position of every (rank, sub-block) segment of this row
    __shared__ int s_segbad;
    extern __shared__ float s_pr[];   // the probabilities of the row's candidates, list order (up to 32768)
    const int b = blockIdx.x, t = threadIdx.x, lane = t & 31, w = t >> 5;
    const float denom = f_denom(stat2, S, b);
    const float bound = f_bound_e(stat2, S, b, denom, top_k, top_p);
    bool ok_row = bound > 0.f;
    const int nseg = world * S;
    // the segment counts are fetched by as many threads at once, then prefixed by one
    if (t < nseg) s_segoff[t + 1] = gath_cnt[(size_t)(t / S) * rstride + (size_t)b * S + (t % S)];
    __syncthreads();
    if (t == 0) {
        uint32_t run = 0;
        int bad = 0;
        for (int i = 0; i < nseg; i++) {
            const uint32_t c = s_segoff[i + 1];
            if (c > (uint32_t)seg) bad = 1;
            s_segoff[i] = run;
            run += min(c, (uint32_t)seg);
        }
        s_segoff[nseg] = run;
        s_segbad = bad;
    }
    __syncthreads();
    const uint32_t M = s_segoff[nseg];
    if (s_segbad) ok_row = false;
    // flat position -> (rank, sub-block, entry); each thread owns a contiguous block of q positions (keeps list order)
    const uint32_t q = (M + kVpThreads - 1) / kVpThreads;
    const uint32_t p0 = min((uint32_t)t * q, M), p1 = min(p0 + q, M);
    auto entry_in = [&](int i, uint32_t pos, float& pr, uint32_t& col) {     // pos lies in segment i
        const uint32_t* e = gath + (size_t)(i / S) * rstride + ((((size_t)b * S) + (i % S)) * seg + (pos - s_segoff[i])) * 2;
        pr = __uint_as_float(e[0]) / denom;
        col = e[1];
    };
    auto entry = [&](uint32_t pos, float& pr, uint32_t& col) {
        int i = 0;
        while (i + 1 < nseg && pos >= s_segoff[i + 1]) i++;
        entry_in(i, pos, pr, col);
    };
    // every probability > bound / denom is on the list (division is monotone; an element just below the bound may
    // round to the same quotient, hence strictly); 16-ary search over that range; the set at its lower end must
    // already fail the test, else the list is too thin
    const uint32_t beta_p = __float_as_uint(bound / denom);
    uint32_t left = beta_p + 1u, right = 0x3f800001u;
    {
        // one look-up and division per candidate (the rounds read shared memory); eight loads in flight at a time
        int i = 0;
        for (uint32_t base = p0; base < p1; base += 8u) {
            uint32_t raw[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const uint32_t pos = base + (uint32_t)u;
                raw[u] = 0u;
                if (pos < p1) {
                    while (i + 1 < nseg && pos >= s_segoff[i + 1]) i++;
                    raw[u] = gath[(size_t)(i / S) * rstride + ((((size_t)b * S) + (i % S)) * seg + (pos - s_segoff[i])) * 2];
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (base + (uint32_t)u < p1) s_pr[base + (uint32_t)u] = __uint_as_float(raw[u]) / denom;
        }
    }
    // The rounds only look at the candidates that still lie in [left, right): those at or above `right` are in every
    // later set (their count and mass are carried), those below `left` in none.  A thread owns at most 32 positions
    // (M <= 32768), so a bit mask names its live ones; three quarters and more drop out per round.  Once nothing is left
    // inside the bracket every further pivot sees the set of `right`, passes, and `left` stays: the loop ends there.
    // (Lists of more than 32768 entries -- more than 16 ranks -- keep every position live and carry nothing.)
    const bool masked = q <= 32u;
    uint32_t live = 0u;
    float left_cnt, base_cnt = 0.f, base_mass = 0.f;
    {
        float v[2] = {0.f, 0.f};
        for (uint32_t pos = p0; pos < p1; pos++) {
            const float pr = s_pr[pos];
            if (__float_as_uint(pr) >= left) { v[0] += 1.f; v[1] += pr; if (masked) live |= 1u << (pos - p0); }
        }
        f_block_sums<2>(v, sh);
        const bool okl = (v[0] < top_k) && (v[1] < top_p);
        if (okl) ok_row = false;
        left_cnt = v[0];
    }
    for (int round = 0; round < RS_VP_ROUNDS && right - left > 1u && left_cnt > base_cnt; round++) {
        uint32_t piv[kVpPivots];
        vp_pivots(left, right, piv);
        float v[30];
#pragma unroll
        for (int j = 0; j < 30; j++) v[j] = 0.f;
        auto tally = [&](const float pr) {
            const uint32_t pb = __float_as_uint(pr);
#pragma unroll
            for (int j = 0; j < kVpPivots; j++)
                if (pb >= piv[j]) { v[2 * j] += 1.f; v[2 * j + 1] += pr; }
        };
        if (masked) {
            for (uint32_t m = live; m; m &= m - 1u) tally(s_pr[p0 + (uint32_t)(__ffs(m) - 1)]);
        } else {
            for (uint32_t pos = p0; pos < p1; pos++) tally(s_pr[pos]);
        }
        f_block_sums30(v, sh);
        uint32_t nl = left, nr = right;
        float ncl = left_cnt, nbc = base_cnt, nbm = base_mass;
        bool found = false;
#pragma unroll
        for (int j = 0; j < kVpPivots; j++) {
            const float cj = base_cnt + v[2 * j], mj = base_mass + v[2 * j + 1];
            const bool okj = (cj < top_k) && (mj < top_p);
            if (!okj) { nl = piv[j]; ncl = cj; }
            else if (!found) { nr = piv[j]; nbc = cj; nbm = mj; found = true; }
        }
        left = nl; right = nr;
        left_cnt = ncl;
        if (!masked) continue;      // every position stays live: the sums are whole sums, nothing is carried
        base_cnt = nbc; base_mass = nbm;
        uint32_t keep = 0u;
        for (uint32_t m = live; m; m &= m - 1u) {
            const int i = __ffs(m) - 1;
            const uint32_t pb = __float_as_uint(s_pr[p0 + (uint32_t)i]);
            if (pb >= left && pb < right) keep |= 1u << i;
        }
        live = keep;
    }
    const float thr = __uint_as_float(left);
    float tl[3] = {0.f, 0.f, 0.f};
    for (uint32_t pos = p0; pos < p1; pos++) {
        const float pr = s_pr[pos];
        if (pr > thr) { tl[0] += 1.f; tl[1] += pr; }
        if (pr == thr) tl[2] += 1.f;
    }
    f_block_sums<3>(tl, sh);
    const float gt4[4] = {tl[0], tl[1], tl[2], 0.f};
    const float comp = vp_comp(gt4, thr, top_k, use_p ? top_p : 0.f, use_p != 0);
    // weights in list order; block scan; the first position whose running weight reaches u * total
    float wsum = 0.f;
    for (uint32_t pos = p0; pos < p1; pos++) wsum += vp_weight_of(s_pr[pos], thr, comp);
    const float incl = warp_scan_desc(wsum, lane);
    if (lane == 31) s_scan[w] = incl;
    if (t == 0) s_hit = 0x7fffffff;
    __syncthreads();
    float pre = 0.f, total = 0.f;
    for (int k = 0; k < 32; k++) { if (k < w) pre += s_scan[k]; total += s_scan[k]; }
    RngWords rng;
    {
        const uint4* st = reinterpret_cast<const uint4*>(states + (long long)b * RS_STATE_BYTES);
        rng.ctr = st[0]; rng.block = st[1]; rng.key_pos = st[2];
    }
    uint32_t r0, r1, r4[4];
    rng_peek2(rng, r0, r1, r4);
    const float target = total * u01(r0);
    float run = pre + incl - wsum;   // weight before this thread's block
    int last_kept = -1;
    for (uint32_t pos = p0; pos < p1; pos++) {
        const float wv = vp_weight_of(s_pr[pos], thr, comp);
        if (wv > 0.f) {
            run += wv;
            last_kept = (int)pos;
            if (target <= run) { atomicMin(&s_hit, (int)pos); break; }
        }
    }
    __syncthreads();
    if (s_hit == 0x7fffffff) {   // rounding only: the last kept position
        __syncthreads();
        if (t == 0) s_hit = -1;
        __syncthreads();
        if (last_kept >= 0) atomicMax(&s_hit, last_kept);
        __syncthreads();
    }
    if (t == 0) {
        int id = 0;
        if (s_hit >= 0 && M > 0) {
            float pr; uint32_t col;
            entry((uint32_t)s_hit, pr, col);
            id = (int)col;
        } else {
            ok_row = false;
        }
        ids[b] = id + 1;
        valid[b] = ok_row ? 1 : 0;
        if (!ok_row) atomicAnd(valid + B, 0);
    }
}

// every rank advances its replica of the RNG states by one block (after a fast-protocol call that was valid)
__global__ void vpf_advance_kernel(unsigned char* states, int B, const int* gate) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B || *gate == 0) return;
    uint4* st = reinterpret_cast<uint4*>(states + (long long)b * RS_STATE_BYTES);
    const uint4 nctr = ctr_next(st[0]);
    const uint4 key = st[2];
    st[0] = nctr;
    st[1] = philox4x32_10(nctr, key.x, key.y);
}

struct VpfLayout { size_t stat1, stat2, send, send_cnt, gath, gath_cnt, ids, valid, total; };
static VpfLayout vpf_layout(long long B, int world, int S) {
    const int lmax = f_lmax(world);
    VpfLayout l;
    size_t o = 0;
    auto take = [&](size_t n) { size_t at = o; o += (n + 63) & ~(size_t)63; return at; };
    l.stat1 = take((size_t)B * S);
    l.stat2 = take((size_t)B * S * kFStat2);
    l.send = take((size_t)B * lmax * 2);                 // S segments of lmax / S entries per row
    l.send_cnt = take((size_t)B * S);                    // one count per segment, directly behind the lists:
    const size_t block = o - l.send;                     // the two travel as one block in one all-gather
    l.gath = take((size_t)world * block);                // rank r's block at gath + r * block
    l.gath_cnt = l.gath + (l.send_cnt - l.send);         // rank 0's counts; rank r's are r * block further on
    l.ids = take(B);
    l.valid = take(B + 1);   // per-row flags, then one flag for the whole call
    l.total = o;
    return l;
}
// sub-blocks per row: enough CTAs to fill the GPU, but every thread keeps >= 16 float4 groups (a thread's
// candidate slots are sized for a sparse sample of a long stripe)
static int vpf_subblocks(long long B, long long n) {
    long long S = 296 / (B > 0 ? B : 1);
    const long long by_work = (n / 4) / (1024 * 16);
    if (S > by_work) S = by_work;
    return S < 1 ? 1 : (S > kFMaxSub ? kFMaxSub : (int)S);
}

}  // namespace rs

extern "C" {

size_t rs_vp_workspace_bytes(int64_t B, int32_t world) {
    if (B <= 0 || world <= 0) return 0;
    return (rs::vp_layout(B, world).total + rs::vpf_layout(B, world, rs::kFMaxSub).total) * sizeof(float);
}

int rs_vp_fast_layout(int64_t B, int64_t V_local, int32_t world, int64_t offsets_floats[11]) {
    if (B <= 0 || world <= 0 || !offsets_floats) return RS_ERR_BATCH;
    const size_t base = rs::vp_layout(B, world).total;
    const int S = rs::vpf_subblocks(B, V_local);
    const rs::VpfLayout l = rs::vpf_layout(B, world, S);
    const size_t o[10] = {l.stat1, l.stat2, l.send, l.send_cnt, l.gath, l.gath_cnt, l.ids, l.valid, (size_t)S, (size_t)rs::f_lmax(world)};
    for (int i = 0; i < 8; i++) offsets_floats[i] = (int64_t)(base + o[i]);
    offsets_floats[8] = (int64_t)o[8];
    offsets_floats[9] = (int64_t)o[9];
    offsets_floats[10] = (int64_t)rs::kFStat2;
    return RS_OK;
}

int rs_vp_layout(int64_t B, int32_t world, int64_t offsets_floats[6]) {
    if (B <= 0 || world <= 0 || !offsets_floats) return RS_ERR_BATCH;
    const rs::VpLayout l = rs::vp_layout(B, world);
    offsets_floats[0] = (int64_t)l.gmax; offsets_floats[1] = (int64_t)l.gsum; offsets_floats[2] = (int64_t)l.tallies;
    offsets_floats[3] = (int64_t)l.gtally; offsets_floats[4] = (int64_t)l.weights; offsets_floats[5] = (int64_t)l.ids;
    return RS_OK;
}

static int vp_tile_common(const rs_vp_call* c, float** stat1, int** all_valid, int* S_out, float* scale) {
    using namespace rs;
    if (!c) return RS_ERR_POINTER;
    const int64_t B = c->B, n = c->V_local, V = c->V_global;
    if (!(V > 0 && V <= 1048576 && V % 4 == 0) || !(n > 0 && n <= V) || n % 4 != 0 || n * (int64_t)c->world != V) return RS_ERR_VOCAB;
    if (!(B > 0) || c->world <= 0 || c->rank < 0 || c->rank >= c->world) return RS_ERR_BATCH;
    if (!(c->temperature >= 0.001 && c->temperature <= 1000)) return RS_ERR_TEMPERATURE;
    if (!c->workspace || ((uintptr_t)c->workspace & 15)) return RS_ERR_POINTER;
    const int S = vpf_subblocks(B, n);
    const VpfLayout f = vpf_layout(B, c->world, S);
    float* fw = (float*)c->workspace + vp_layout(B, c->world).total;
    *stat1 = fw + f.stat1;
    *all_valid = (int*)(fw + f.valid) + B;
    *S_out = S;
    *scale = (float)(1.4426950408889634074 / c->temperature);
    return RS_OK;
}

int rs_vp_tile_begin(const rs_vp_call* c) {
    float* stat1; int* all_valid; int S; float scale;
    const int rc = vp_tile_common(c, &stat1, &all_valid, &S, &scale);
    if (rc) return rc;
    const int n = (int)(c->B * S);
    rs::vpf_tile_begin_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)c->stream>>>(stat1, n, all_valid);
    return cudaGetLastError() == cudaSuccess ? RS_OK : RS_ERR_CUDA;
}

int rs_vp_tile_max(const rs_vp_call* c, const float* tile_device, int64_t ld, int64_t col_begin, int64_t ncols) {
    float* stat1; int* all_valid; int S; float scale;
    const int rc = vp_tile_common(c, &stat1, &all_valid, &S, &scale);
    if (rc) return rc;
    if (!tile_device || ((uintptr_t)tile_device & 3)) return RS_ERR_POINTER;
    if (ncols <= 0 || col_begin < 0 || col_begin + ncols > c->V_local || ld < ncols) return RS_ERR_VOCAB;
    const float* pen = c->penalties ? c->penalties + col_begin : nullptr;
    dim3 grid((unsigned)((ncols + 4095) / 4096), (unsigned)c->B);
    rs::vpf_tile_max_kernel<<<grid, 256, 0, (cudaStream_t)c->stream>>>(tile_device, (long long)ld, pen, (long long)c->V_local,
                                                                       (int)ncols, scale, S, stat1);
    return cudaGetLastError() == cudaSuccess ? RS_OK : RS_ERR_CUDA;
}

int rs_vp_stage(const rs_vp_call* c, int32_t stage, int32_t round) {
    using namespace rs;
    if (!c) return RS_ERR_POINTER;
    const int64_t B = c->B, T = c->T, n = c->V_local, V = c->V_global;
    if (!(V > 0 && V <= 1048576 && V % 4 == 0) || !(n > 0 && n <= V)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0) || c->world <= 0 || c->rank < 0 || c->rank >= c->world) return RS_ERR_BATCH;
    // The shard kernels read float4 groups at row_base + g: every row of the shard must start on a 16-byte boundary,
    // and the shards must tile the vocabulary in rank order (the finishing kernel reports GLOBAL column ids).
    if (n % 4 != 0 || n * (int64_t)c->world != V || c->col0 != (int64_t)c->rank * n) return RS_ERR_VOCAB;
    if (!(c->temperature >= 0.001 && c->temperature <= 1000)) return RS_ERR_TEMPERATURE;
    if (!c->logits || !c->states || !c->workspace) return RS_ERR_POINTER;
    if (((uintptr_t)c->logits & 15) || ((uintptr_t)c->penalties & 15) || ((uintptr_t)c->workspace & 15) ||
        ((uintptr_t)c->states & 15))
        return RS_ERR_POINTER;
    int64_t top_k = c->top_k;
    double top_p = c->top_p;
    if (top_k <= 0 || top_k > V) top_k = V;          // remaps of sampling.cu:1005-1010, on the GLOBAL vocabulary
    if (top_p < 0 || top_p > 1) top_p = 1;
    if (top_p == 0) { top_k = 1; top_p = 1; }
    const int use_p = top_p < 1.0 ? 1 : 0;            // top_p == 1: the mass never limits (sampling.cu:596)
    const float fk = (float)top_k, fp = use_p ? (float)top_p : INFINITY;
    const float scale = (float)(1.4426950408889634074 / c->temperature);
    const VpLayout l = vp_layout(B, c->world);
    float* ws = (float*)c->workspace;
    const float* lg = c->logits + (T - 1) * n;
    const long long stride = (long long)T * n;
    cudaStream_t st = (cudaStream_t)c->stream;
    const unsigned grid = (unsigned)B;
    switch (stage) {
        case RS_VP_MAX:
            vp_max_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax);
            break;
        case RS_VP_SUM:
            vp_sum_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax, ws + l.gsum);
            break;
        case RS_VP_ROUND:
            if (round < 0 || round >= RS_VP_ROUNDS) return RS_ERR_LIMIT;
            vp_round_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax, ws + l.gsum,
                                                         ws + l.tallies, (int)B, round, fk, fp,
                                                         ws + l.tallies + (size_t)round * B * kVpPivots * 2);
            break;
        case RS_VP_TALLY:
            vp_tally_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax, ws + l.gsum,
                                                         ws + l.tallies, (int)B, RS_VP_ROUNDS, fk, fp, ws + l.gtally);
            break;
        case RS_VP_WEIGHT:
            if (cudaMemsetAsync(ws + l.weights, 0, (size_t)B * c->world * sizeof(float), st) != cudaSuccess) return RS_ERR_CUDA;
            vp_weight_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax, ws + l.gsum,
                                                          ws + l.tallies, (int)B, RS_VP_ROUNDS, fk, fp, use_p, ws + l.gtally,
                                                          c->rank, c->world, ws + l.weights);
            break;
        case RS_VP_PICK:
            vp_pick_kernel<<<grid, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, ws + l.gmax, ws + l.gsum,
                                                        ws + l.tallies, (int)B, RS_VP_ROUNDS, fk, fp, use_p, ws + l.gtally,
                                                        ws + l.weights, c->rank, c->world, (unsigned char*)c->states,
                                                        (long long)c->col0, (int*)(ws + l.ids));
            break;
        case RS_VP_PENALTY:
            if (c->penalties) {
                const long long tot = (long long)B * n;
                const int* idsrc = (round == 1) ? (const int*)(ws + l.total + vpf_layout(B, c->world, vpf_subblocks(B, n)).ids)
                                                : (const int*)(ws + l.ids);   // argument `round` == 1 selects the ids of the fast protocol
                vp_penalty_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(
                    c->penalties, (int)n, (int)B, idsrc, (long long)c->col0, (float)c->presence_penalty,
                    (float)c->repetition_penalty, (float)c->penalty_decay,
                    (round == 1) ? (const int*)(ws + l.total + vpf_layout(B, c->world, vpf_subblocks(B, n)).valid) + B : nullptr);
            }
            break;
        case RS_VPF_MAX: case RS_VPF_SUM: case RS_VPF_EXTRACT: case RS_VPF_COMPACT: case RS_VPF_FINISH: case RS_VPF_ADVANCE: {
            const int S = vpf_subblocks(B, n);
            // the finishing kernel's segment table and its live-position masks are sized for 64 segments of a row
            if ((long long)c->world * S > kFMaxSub * 8) return RS_ERR_LIMIT;
            const VpfLayout f = vpf_layout(B, c->world, S);
            const int lmax = f_lmax(c->world);
            float* fw = ws + l.total;
            uint32_t* uw = reinterpret_cast<uint32_t*>(fw);
            if (stage == RS_VPF_MAX)
                vpf_max_kernel<<<grid * S, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, S, fw + f.stat1,
                                                                (int*)(uw + f.valid) + B);
            else if (stage == RS_VPF_SUM)
                vpf_sum_kernel<<<grid * S, kVpThreads, 0, st>>>(lg, stride, c->penalties, (int)n, scale, S, fw + f.stat1,
                                                                fw + f.stat2);
            else if (stage == RS_VPF_EXTRACT) {
                constexpr size_t kExtractSmem = (size_t)kFCap * kVpThreads * sizeof(uint2);
                static bool attr_done_x[64] = {};     // per device
                int dev = 0;
                if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RS_ERR_CUDA;
                if (!attr_done_x[dev]) {
                    if (cudaFuncSetAttribute(vpf_extract_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kExtractSmem) !=
                        cudaSuccess)
                        return RS_ERR_CUDA;
                    attr_done_x[dev] = true;
                }
                vpf_extract_kernel<<<grid * S, kVpThreads, kExtractSmem, st>>>(lg, stride, c->penalties, (int)n, scale, S, fw + f.stat1,
                                                                               fw + f.stat2, fk, fp, lmax / S, uw + f.send,
                                                                               uw + f.send_cnt, (long long)c->col0);
            } else if (stage == RS_VPF_COMPACT) {
                // nothing to do: the extraction writes the ordered list itself (the stage stays for drivers that name it)
                return RS_OK;
            } else if (stage == RS_VPF_FINISH) {
                // the union of the ranks' lists is staged in shared memory: 4 bytes per candidate
                constexpr size_t kFinishSmem = 160 * 1024;
                if ((size_t)lmax * c->world * sizeof(float) > kFinishSmem) return RS_ERR_LIMIT;
                static bool attr_done[64] = {};     // per device
                int dev = 0;
                if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RS_ERR_CUDA;
                if (!attr_done[dev]) {
                    if (cudaFuncSetAttribute(vpf_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFinishSmem) !=
                        cudaSuccess)
                        return RS_ERR_CUDA;
                    attr_done[dev] = true;
                }
                vpf_finish_kernel<<<grid, kVpThreads, (size_t)lmax * c->world * sizeof(float), st>>>((int)B, S, c->world, lmax / S, fw + f.stat1, fw + f.stat2, uw + f.gath,
                                                               uw + f.gath_cnt, f.gath - f.send /* one rank's block */, fk, fp, use_p, (const unsigned char*)c->states,
                                                               (int*)(uw + f.ids), (int*)(uw + f.valid));
            } else
                vpf_advance_kernel<<<(unsigned)((B + 127) / 128), 128, 0, st>>>((unsigned char*)c->states, (int)B,
                                                                                (const int*)(uw + f.valid) + B);
            break;
        }
        default:
            return RS_ERR_LIMIT;
    }
    return cudaGetLastError() == cudaSuccess ? RS_OK : RS_ERR_CUDA;
}

}  // extern "C"
