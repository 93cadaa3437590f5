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
                                  float presence, float repetition, float decay) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * n) return;
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

}  // namespace rs

extern "C" {

size_t rs_vp_workspace_bytes(int64_t B, int32_t world) {
    if (B <= 0 || world <= 0) return 0;
    return rs::vp_layout(B, world).total * sizeof(float);
}

int rs_vp_layout(int64_t B, int32_t world, int64_t offsets_floats[6]) {
    if (B <= 0 || world <= 0 || !offsets_floats) return RS_ERR_BATCH;
    const rs::VpLayout l = rs::vp_layout(B, world);
    offsets_floats[0] = (int64_t)l.gmax; offsets_floats[1] = (int64_t)l.gsum; offsets_floats[2] = (int64_t)l.tallies;
    offsets_floats[3] = (int64_t)l.gtally; offsets_floats[4] = (int64_t)l.weights; offsets_floats[5] = (int64_t)l.ids;
    return RS_OK;
}

int rs_vp_stage(const rs_vp_call* c, int32_t stage, int32_t round) {
    using namespace rs;
    if (!c) return RS_ERR_POINTER;
    const int64_t B = c->B, T = c->T, n = c->V_local, V = c->V_global;
    if (!(V > 0 && V <= 1048576 && V % 4 == 0) || !(n > 0 && n <= V)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0) || c->world <= 0 || c->rank < 0 || c->rank >= c->world) return RS_ERR_BATCH;
    if (!(c->temperature >= 0.001 && c->temperature <= 1000)) return RS_ERR_TEMPERATURE;
    if (!c->logits || !c->states || !c->workspace) return RS_ERR_POINTER;
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
            cudaMemsetAsync(ws + l.weights, 0, (size_t)B * c->world * sizeof(float), st);
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
                vp_penalty_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(
                    c->penalties, (int)n, (int)B, (const int*)(ws + l.ids), (long long)c->col0, (float)c->presence_penalty,
                    (float)c->repetition_penalty, (float)c->penalty_decay);
            }
            break;
        default:
            return RS_ERR_LIMIT;
    }
    return cudaGetLastError() == cudaSuccess ? RS_OK : RS_ERR_CUDA;
}

}  // extern "C"
