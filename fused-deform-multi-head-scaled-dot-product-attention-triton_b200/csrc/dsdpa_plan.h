// Host-side planning: which kernel variant and tile shape a problem runs with.
// Stands where the reference's 81-configuration autotune sits (ops/triton.py:10-25):
// the choice is made from the shape, once, on the host, by a small cost model.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/dsdpa.h"

namespace dsdpa {

constexpr int kPlanSMs = 148;
constexpr int kPlanSmemMax = 232448;
constexpr int kPlanRecBytesPerWarp = 1024;
// Threads bwd_gather_kernel is compiled for (and run with): 16-bit storage keeps 32 accumulators
// and the unpacked operands per lane, which fit 96 registers (640 threads) without spills and
// measured 8% faster than 768 threads at 80; fp32 storage needs fewer registers and runs best at 768.
constexpr int kGatherThreadsNarrow = 640;
constexpr int kGatherThreadsFp32 = 768;
inline int gather_max_threads(int dtype) { return dtype == DSDPA_F32 ? kGatherThreadsFp32 : kGatherThreadsNarrow; }

inline int dtype_size(int dtype) { return dtype == DSDPA_F32 ? 4 : 2; }

struct RowGeom {
    int G;   // lanes per row
    int NG;  // groups per warp
};
inline RowGeom row_geom(int D, int dtype) {
    int vec = D * dtype_size(dtype) / 16;
    RowGeom r;
    r.G = vec < 32 ? vec : 32;
    r.NG = 32 / r.G;
    return r;
}

struct TilePlan {
    bool staged;       // K/V maps of one key view staged in shared memory
    bool priv;         // backward only: dK/dV maps privatised in shared memory
    bool rounded_weights;  // forward, 16-bit storage: DSDPA_FLAG_ROUNDED_WEIGHTS
    int nstage;        // map buffers (staged)
    int nw;            // warps per CTA
    int nq;            // query slots per group (template parameter)
    int tiles;         // tiles per (batch, head)
    int q_per_tile;
    size_t smem;       // dynamic shared memory per CTA
    long long ctas;
};

// Two-pass backward: gather tiles and the layout of its scratch inside the workspace.
struct GatherPlan {
    bool ok;            // the shape can run the two-pass form
    int tpv;            // gather tiles per query view
    int QB;             // queries (pixels of one query view) per gather tile, even
    int gather_threads;
    size_t gather_smem;
    int A;                   // anchors per map, H*(W+1): the lists the index is sorted into
    int nhist;               // histograms (sample-taking warps) of the index builder
    int nslab;               // CTAs that split the map rows of one (batch, head, key view)
    long long gather_ctas;   // B*Hh*V*nslab
    long long segments;      // B * (V*tpv) * V index segments
    int seg_entries;         // index entries reserved per segment
    size_t index_smem;
    // byte offsets inside the workspace (after the fp32 dK/dV accumulators, if any)
    size_t scal_bytes, entries_bytes, sched_bytes, hdr_bytes;
};
GatherPlan plan_gather(const dsdpa_problem& p);

// `backward`: plan for the scatter kernel (it can additionally privatise dK/dV).
TilePlan plan_tiles(const dsdpa_problem& p, bool backward, bool allow_priv);

int validate_problem(const dsdpa_problem* p);

}  // namespace dsdpa
