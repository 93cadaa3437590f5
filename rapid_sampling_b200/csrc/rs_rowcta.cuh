// Launch interface of the row-per-CTA sampler variant (rs_rowcta.cu).
#pragma once
#include <cuda_runtime.h>

namespace rs {

struct Params;

constexpr int kRowCtaFixedSmem = 6400;   // scalars, scan totals, the two exchange boxes and the unordered candidate list ahead of the per-lane lists

// How a row-CTA launch lays out its dynamic shared memory.
struct RowCtaPlan {
    int depth;         // stages of a thread's copy pipeline (each one stripe of logits, plus one of penalties beside it)
    int cached;        // leading stripes that stay on chip as scaled logits between the two passes
    int cap;           // candidate entries per virtual lane
    int stage_bytes;
    int off_cand, off_ring, off_cache;
    int smem_bytes;
};

RowCtaPlan rowcta_plan(int V, bool with_penalties, int sel_rank, int lanes_per_thread, int smem_budget);
// lanes_per_thread: 2 (512 threads per row; batches that leave an SM to one row) or 4 (256 threads; two rows per SM)
// dependent: launch with programmatic stream serialization (the kernel waits for its predecessor itself)
int rowcta_launch(const Params& p, const RowCtaPlan& pl, int lanes_per_thread, cudaStream_t stream, int smem_optin, bool dependent);

}  // namespace rs
