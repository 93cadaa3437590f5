// Device-side building blocks of the sampler: counter-based RNG, fixed-order warp primitives,
// cluster / bulk-copy PTX wrappers.  sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdint.h>

namespace rs {

constexpr int kLanes = 1024;  // virtual lanes per row: lane t owns float4 groups t, t+1024, ...
constexpr int kWarps = 32;    // virtual warps per row (32 consecutive lanes)

// ------------------------------------------------------------------ RNG ------------------
// Philox4x32-10 (Salmon et al., SC'11).  The 64-byte per-row state keeps the field order of
// curandStatePhilox4_32_10_t (the reference's RAND, sampling.cu:9) so that states made by
// either library continue the same stream in the other.
struct RngWords {   // the three 16-byte words of the state that matter
    uint4 ctr;      // 128-bit counter; the row index sits in .z/.w (subsequence)
    uint4 block;    // cached output of the current counter
    uint4 key_pos;  // key.x, key.y, pos (index of the next unused word of block), unused
};

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c;
}

__device__ __forceinline__ uint4 ctr_next(uint4 c) {
    if (++c.x == 0) if (++c.y == 0) if (++c.z == 0) ++c.w;
    return c;
}

// u32 -> (0, 1]: x * 2^-32 + 2^-33 in fp32 (the product is exact, so fusing changes nothing).
__device__ __forceinline__ float u01(uint32_t x) {
    return __uint2float_rn(x) * 2.3283064365386963e-10f + 1.1641532182693481e-10f;
}

// First two words of the next 4-word draw, without touching the stored state.
__device__ __forceinline__ void rng_peek2(const RngWords& s, uint32_t& r0, uint32_t& r1, uint32_t out4[4]) {
    const uint32_t pos = s.key_pos.z & 3u;
    uint32_t w[8] = {s.block.x, s.block.y, s.block.z, s.block.w, 0, 0, 0, 0};
    if (pos != 0) {  // only states that were advanced by single-word draws elsewhere
        const uint4 nb = philox4x32_10(ctr_next(s.ctr), s.key_pos.x, s.key_pos.y);
        w[4] = nb.x; w[5] = nb.y; w[6] = nb.z; w[7] = nb.w;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t v = w[i];
#pragma unroll
        for (int q = 1; q < 4; q++) v = (pos == (uint32_t)q) ? w[i + q] : v;
        out4[i] = v;
    }
    r0 = out4[0];
    r1 = out4[1];
}

// ------------------------------------------------------- fixed-order primitives ----------
// Inf/NaN sanitiser of the reference (sampling.cu:131-134): NaN -> 0, +-Inf -> +-FLT_MAX.
__device__ __forceinline__ float sanitize(float x) {
    const float y = isnan(x) ? 0.0f : x;
    return isinf(y) ? copysignf(FLT_MAX, y) : y;
}

// xor butterfly, offsets 16,8,4,2,1: every lane ends with the same balanced-tree value
// (association of sampling.cu:11-17).
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Inclusive scan with DESCENDING shuffle offsets (sampling.cu:48-58).  For non-negative fp32
// this order makes the prefix sequence non-decreasing, which an ascending order does not.
__device__ __forceinline__ float warp_scan_desc(float v, int lane) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

// ------------------------------------------------------------- PTX wrappers --------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Programmatic dependent launch (kernels launched with cudaLaunchAttributeProgrammaticStreamSerialization).
// wait: returns once every kernel this one depends on has completed and its memory operations are visible (at once
// for an ordinary launch).  may_launch: lets the next kernel of the stream be scheduled early; it runs up to its own
// wait while this one is still working.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// Remote 4-byte store whose completion is counted on an mbarrier of the destination CTA.
__device__ __forceinline__ void st_async_u32(uint32_t addr, uint32_t v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];" ::"r"(addr), "r"(v),
                 "r"(remote_bar)
                 : "memory");
}
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
                 "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
                 : "memory");
}
__device__ __forceinline__ void st_async_v2(uint32_t addr, uint32_t a, uint32_t b, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(addr), "r"(a),
                 "r"(b), "r"(remote_bar)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a bounded,
// hardware-defined time) and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// 1-D bulk async copy global -> this CTA's shared memory, completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

}  // namespace rs
