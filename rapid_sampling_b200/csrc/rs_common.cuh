// Pieces shared by the sampler kernels: launch parameters, the per-row argument record, the strided row view
// used by the whole-row search, and the element-wise arithmetic (scaled / penalised logits) that every variant
// must compute with the same operations in the same order.  sm_100a only.
#pragma once
#include "rs_device.cuh"
#include "../../include/rapid_sampling_b200.h"

namespace rs {

enum Kind : int { kTopP = 0, kGeneral = 1, kRepetition = 2 };

struct Params {
    const void* logits;      // already offset to position T-1 of row 0; fp32, fp16 or bf16 (dtype)
    int dtype;               // RS_DTYPE_F32 / F16 / BF16 of the logits
    long long row_stride;    // elements between consecutive rows (T*V)
    float* penalties;        // (B,V) or null
    unsigned char* states;   // B*64
    int* out;                // B
    float* scratch;          // B*V floats (global-row variant only)
    float* dbg_probs;        // optional (B,V)
    rs_trace* dbg_trace;     // optional B
    int* status;             // device status word
    int* status_mirror;      // optional: a word of pinned host memory the device can write (zero-copy), or null
    uint32_t wait_polls;     // polls after which a bounded wait gives up
    int B, V, kind, top_k;
    int sel_rank;            // 0 = no candidate shortcut; else rank of the per-warp thread maximum used as bound
    int cand_slots;          // float4 slots per lane of the candidate buffer (shared-memory variant)
    float scale, top_p, presence, repetition, decay;
    const struct RowArgs* rows;   // per-row parameters (ROWP kernels only), else null
    float* out_prob;         // optional B: probability of the sampled id (ROWP kernels only)
    float* out_kept;         // optional B: kept probability mass the id was drawn from (ROWP kernels only)
    int quick;               // 1: try the one-warp search on integer masses first; 0 (test instrumentation): exact search only
};

// Normalised parameters of one row, made on the device from the caller's per-row tensors.
struct __align__(32) RowArgs {
    int kind, top_k, sel_rank, pad0;
    float scale, top_p, pad1, pad2;
};

// shared-memory map (bytes)
constexpr int kXWords = 10;                      // words each warp contributes to an exchange
template <int N> struct Packets { static constexpr int value = N; };   // 16-byte packets of an exchange record
constexpr int kXStride = 12;                     // words between two warps' records in a mailbox (16-byte aligned records)
constexpr int kMboxOff = 0;                      // 2 buffers of [32 warps][kXStride] words
constexpr int kMboxBuf = kXStride * 32 * 4;
constexpr int kMiscOff = 2 * kMboxBuf;           // mbarriers, small scalars, 32 warp totals
constexpr int kQuickCap = 512;                   // longest candidate list the one-warp search takes
constexpr int kQuickOff = kMiscOff + 256;        // the row's candidates as one unordered list of (bits of p, p in units of 2^-30)
constexpr int kSlabOff = kQuickOff + kQuickCap * 8;
constexpr uint32_t kDefaultWaitPolls = 1u << 22;

__host__ __device__ constexpr int slab_bytes(int V, int C) { return ((V / 4 + 1023) / 1024) * (1024 / C) * 16; }

template <int C, bool SMEM>
struct Row {
    static constexpr int L = kLanes / C;
    float4* slab;
    int t, tg;
    __device__ __forceinline__ float4 ld(int s) const { return SMEM ? slab[s * L + t] : slab[s * kLanes + tg]; }
    __device__ __forceinline__ void st(int s, float4 v) const {
        if (SMEM) slab[s * L + t] = v; else slab[s * kLanes + tg] = v;
    }
};

// Probability of one element, exactly as the streaming passes compute it.
__device__ __forceinline__ float scaled_logit(float l, float pen, bool rep, float scale) {
    return rep ? sanitize((sanitize(l) - pen) * scale) : sanitize(l * scale);
}

// One search pass over this lane's list in the slab: ordered masses and counts at three pivots
// (f[3] is ignored here); optionally keeps only elements >= keepf (in place, order preserved, tail
// padded with -1).  Counts are returned packed: c01 = n(f0) | n(f1) << 16, c23 = n(f2).
template <int C, bool SMEM, bool COMPACT>
__device__ __forceinline__ void slab_pass(const Row<C, SMEM>& row, int& n, const float (&f)[4], float keepf, float (&m)[4],
                                          uint32_t& c01, uint32_t& c23) {
    uint32_t cy = 0, cz = 0, cw = 0;
    float my = 0.f, mz = 0.f, mw = 0.f;
    const float py = f[0], pz = f[1], pw = f[2];
    const int slots = (n + 3) >> 2;
    float b0 = -1.f, b1 = -1.f, b2 = -1.f, b3 = -1.f;
    int q = 0;
#pragma unroll ((SMEM || COMPACT || C > 1) ? 2 : 4)
    for (int s = 0; s < slots; s++) {
        const float4 v = row.ld(s);
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p = e[j];
            if (p >= py) { cy++; my += p; }
            if (p >= pz) { cz++; mz += p; }
            if (p >= pw) { cw++; mw += p; }
            if (COMPACT) {
                if (p >= keepf) {
                    const int k = q & 3;
                    b0 = (k == 0) ? p : b0;
                    b1 = (k == 1) ? p : b1;
                    b2 = (k == 2) ? p : b2;
                    b3 = (k == 3) ? p : b3;
                    q++;
                    if ((q & 3) == 0) {
                        row.st((q >> 2) - 1, make_float4(b0, b1, b2, b3));
                        b0 = b1 = b2 = b3 = -1.f;
                    }
                }
            }
        }
    }
    if (COMPACT) {
        if (q & 3) row.st(q >> 2, make_float4(b0, b1, b2, b3));
        n = q;
    }
    m[0] = my; m[1] = mz; m[2] = mw; m[3] = 0.f;
    c01 = cy | (cz << 16);
    c23 = cw;
}

// ---- the cutoff search of a whole row's candidate list in ONE warp, on integer masses ---------------------------
// The reference's loop only ever asks whether a mass is below or above top_p (sampling.cu:598, :618-651).  `list`
// holds every candidate of the row as (bits of p, p in units of 2^-30), in any order: the sum of the admitted
// entries' second words is exact up to half a unit per entry and does not depend on the order.  The reference's fp32
// value differs from the true sum by at most one rounding per addition on the longest path (`depth`: the entries of
// one lane, 5 in the warp tree, 31 over the warps).  Outside that margin around top_p the answer is certain and the
// loop is replayed here -- same pivots, same tests, same bracket updates -- without any exchange; inside it (unless a
// count decides the test anyway) the verdict is 0 and the caller runs the exact search from the start.
// Pivots at or below beta_p are answered by the set {p > beta_p}, as in the exact search on a candidate list.
// All 32 lanes call this with the same arguments; `list` must be readable up to the next multiple of 256 entries
// (entries from n on are overwritten with "never admitted").
// FREEZE: once the sets at `left` and at `right` differ by at most one entry, the remaining rounds are replayed from the
// carried values without reading the list (pays where rounds are many; costs registers).
// Verdict: 1 settled (left / right / rounds are the reference's), 2 the list cannot settle the cutoff, 0 undecided.
template <bool FREEZE>
__device__ __forceinline__ int quick_search(uint2* list, const uint32_t n, const int lane, const int depth, const bool use_cnt,
                                            const uint32_t top_k, const float top_p, const uint32_t beta_p, const float pmin,
                                            const float pmax, const uint32_t V, uint32_t& left, uint32_t& right, uint32_t& rounds) {
    constexpr unsigned FULLW = 0xffffffffu;
    for (uint32_t i = n + (uint32_t)lane; i < ((n + 255u) & ~255u); i += 32u) list[i] = make_uint2(0u, 0u);
    __syncwarp();
    const uint32_t margin = (uint32_t)(depth * 66 + kQuickCap / 2 + 8);
    const uint32_t tp_lo = __float2uint_rd(top_p * 1073741824.f), tp_hi = __float2uint_ru(top_p * 1073741824.f);
    const uint32_t ustar = beta_p + 1u;
    uint32_t l_left = __float_as_uint(pmin), l_right = __float_as_uint(pmax) + 1u, l_rounds = 0u;
    // what the loop carries: the count at `left` and whether its mass is above top_p (the reference starts from the
    // whole row and mass 1); kept beside it for the replay below: the same for `right` (nothing lies above pmax)
    uint32_t cnt_x = V, cnt_r = 0u;
    bool gt_x = 1.0f > top_p, lt_x = 1.0f < top_p, gt_r = false, lt_r = 0.0f < top_p;
    bool have_x = false;                 // cnt_x counts list entries (left came from an evaluated pivot)
    bool frozen = false;                 // at most one entry is left in [max(left, u*), right): no more scans
    uint32_t v_bits = 0u;                // that entry (0: none; every evaluation point is above 0)
    int verdict = 1;
    for (;;) {
        const bool go = use_cnt ? (cnt_x > top_k || gt_x) : gt_x;
        if (!(go && l_left < l_right - 1u) || l_rounds >= 64u) break;
        l_rounds++;
        const uint32_t pz = (l_left + l_right) >> 1, py = (l_left + pz) >> 1, pwv = (pz + l_right) >> 1;
        const uint32_t pv[3] = {py, pz, pwv};
        const uint32_t ev[3] = {max(py, ustar), max(pz, ustar), max(pwv, ustar)};
        uint32_t cnt[3];
        bool lt[3], gt[3], unsure = false;
        if (FREEZE && !frozen && have_x && cnt_x - cnt_r <= 1u) {
            // The sets at `left` and at `right` differ by at most one entry, v: an evaluation point at or below v sees
            // the set of `left`, one above v the set of `right`; the remaining rounds need no data.
            frozen = true;
            if (cnt_x != cnt_r) {
                uint32_t m = 0u;
                for (uint32_t i0 = 0u; i0 < n; i0 += 256u) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const uint32_t e = list[i0 + (uint32_t)(i * 32 + lane)].x;
                        m = (e < l_right) ? max(m, e) : m;
                    }
                }
                v_bits = __reduce_max_sync(FULLW, m);
            }
        }
        if (FREEZE && frozen) {
#pragma unroll
            for (int i = 0; i < 3; i++) {
                const bool at_x = ev[i] <= v_bits;
                cnt[i] = at_x ? cnt_x : cnt_r;
                lt[i] = at_x ? lt_x : lt_r;
                gt[i] = at_x ? gt_x : gt_r;
            }
        } else {
            uint32_t c0 = 0u, c1 = 0u, c2 = 0u, q0 = 0u, q1 = 0u, q2 = 0u;
            for (uint32_t i0 = 0u; i0 < n; i0 += 256u) {
                uint2 en[8];
#pragma unroll
                for (int i = 0; i < 8; i++) en[i] = list[i0 + (uint32_t)(i * 32 + lane)];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (en[i].x >= ev[0]) { c0++; q0 += en[i].y; }
                    if (en[i].x >= ev[1]) { c1++; q1 += en[i].y; }
                    if (en[i].x >= ev[2]) { c2++; q2 += en[i].y; }
                }
            }
            cnt[0] = __reduce_add_sync(FULLW, c0); cnt[1] = __reduce_add_sync(FULLW, c1); cnt[2] = __reduce_add_sync(FULLW, c2);
            const uint32_t qm[3] = {__reduce_add_sync(FULLW, q0), __reduce_add_sync(FULLW, q1), __reduce_add_sync(FULLW, q2)};
#pragma unroll
            for (int i = 0; i < 3; i++) {
                lt[i] = qm[i] + margin < tp_lo;
                gt[i] = qm[i] > tp_hi + margin;
                unsure = unsure || (!lt[i] && !gt[i] && !(use_cnt && cnt[i] > top_k));
            }
        }
        if (unsure) { verdict = 0; break; }
        bool ok[3], bad = false;
#pragma unroll
        for (int i = 0; i < 3; i++) {
            const bool below = pv[i] <= beta_p;
            const bool exceeds = (use_cnt && cnt[i] > top_k) || gt[i];
            const bool pass = (!use_cnt || cnt[i] < top_k) && lt[i];
            ok[i] = !below && pass;
            bad = bad || (below && !exceeds);
        }
        if (bad) { verdict = 2; break; }
        const bool s0 = ok[0], s1 = !s0 && ok[1], s2 = !s0 && !s1 && ok[2];
        const uint32_t nl = s0 ? l_left : s1 ? pv[0] : s2 ? pv[1] : pv[2];
        const uint32_t nr = s0 ? pv[0] : s1 ? pv[1] : s2 ? pv[2] : l_right;
        const uint32_t ncx = s0 ? cnt_x : s1 ? cnt[0] : s2 ? cnt[1] : cnt[2];
        const bool ngx = s0 ? gt_x : s1 ? gt[0] : s2 ? gt[1] : gt[2];
        l_left = nl; l_right = nr;
        cnt_x = ncx; gt_x = ngx;
        if (FREEZE) {
            const bool nlx = s0 ? lt_x : s1 ? lt[0] : s2 ? lt[1] : lt[2];
            const uint32_t ncr = s0 ? cnt[0] : s1 ? cnt[1] : s2 ? cnt[2] : cnt_r;
            const bool ngr = s0 ? gt[0] : s1 ? gt[1] : s2 ? gt[2] : gt_r;
            const bool nlr = s0 ? lt[0] : s1 ? lt[1] : s2 ? lt[2] : lt_r;
            have_x = have_x || !s0;
            lt_x = nlx; cnt_r = ncr; gt_r = ngr; lt_r = nlr;
        }
    }
    if (verdict == 1 && !(l_left > beta_p)) verdict = 2;
    left = l_left; right = l_right; rounds = l_rounds;
    return verdict;
}

// Sanitised scaled logit with the common case (finite product) kept to a multiply and a compare.
__device__ __forceinline__ float scaled_fast(float l, float scale) {
    const float x = l * scale;
    return (fabsf(x) <= FLT_MAX) ? x : sanitize(x);
}
// The rare path, kept out of line so that the streaming loops stay short.
__device__ __forceinline__ float4 sanitize4(float4 v) {
    return make_float4(sanitize(v.x), sanitize(v.y), sanitize(v.z), sanitize(v.w));
}
// Four scaled logits; a single test per group finds any Inf / NaN product (x * 0 is NaN exactly for those).
__device__ __forceinline__ float4 scaled4(float4 l, float scale) {
    float4 v = make_float4(l.x * scale, l.y * scale, l.z * scale, l.w * scale);
    const float probe = fmaf(v.w, 0.f, fmaf(v.z, 0.f, fmaf(v.y, 0.f, v.x * 0.f)));
    if (probe != probe) v = sanitize4(v);
    return v;
}
// Four penalised scaled logits, sanitize((sanitize(l) - pen) * scale).  If the plain product is finite, the logit
// was finite too (an Inf / NaN logit keeps the product non-finite for any finite or non-finite penalty), both
// sanitisers were identities and the product is the result; anything else takes the exact formula.
__device__ __forceinline__ float4 scaled4_rep(float4 l, float4 q, float scale) {
    float4 v = make_float4((l.x - q.x) * scale, (l.y - q.y) * scale, (l.z - q.z) * scale, (l.w - q.w) * scale);
    const float probe = fmaf(v.w, 0.f, fmaf(v.z, 0.f, fmaf(v.y, 0.f, v.x * 0.f)));
    if (probe != probe)
        v = make_float4(scaled_logit(l.x, q.x, true, scale), scaled_logit(l.y, q.y, true, scale),
                        scaled_logit(l.z, q.z, true, scale), scaled_logit(l.w, q.w, true, scale));
    return v;
}
// Appends the candidates of one float4 group to the lane's list (rare; out of line).
__device__ __forceinline__ void append_candidates(float4 v, float beta_e, float* list, int stride4, int cap, int& nc, int& ns) {
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (e[j] >= beta_e) {
            if (nc < cap) list[(nc >> 2) * stride4 + (nc & 3)] = e[j];
            nc++;
            ns += (e[j] > beta_e) ? 1 : 0;
        }
    }
}


}  // namespace rs
