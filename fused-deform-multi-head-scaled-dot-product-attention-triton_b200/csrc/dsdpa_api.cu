// C ABI of libdeform_sdpa.so: argument checks, planning, launches, status reporting.
// Declarations and the reference interfaces they replace are in include/dsdpa.h.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>

#include "dsdpa_launch.cuh"

namespace dsdpa {

// Written by a kernel whose bounded wait ran out (one word per device that loads the module).
__device__ int g_error_word;

static thread_local int t_last_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};

static int cuda_fail(cudaError_t e) {
    t_last_cuda_error = (int)e;
    (void)cudaGetLastError();  // clear the sticky-free error state
    return DSDPA_ERR_CUDA;
}
// For the library's other translation units: record a failed CUDA call the same way.
int report_cuda_failure(int cuda_error) { return cuda_fail((cudaError_t)cuda_error); }

// The bounded wait on its own, for the self-test entry: one warp waits on an mbarrier nobody
// ever completes, gives up after `polls` polls, records that and returns.
__global__ void __launch_bounds__(32) selftest_wait_kernel(unsigned polls, int* err) {
    __shared__ __align__(8) unsigned long long bar_storage;
    const uint32_t bar = smem_addr(&bar_storage);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    (void)mbar_wait_bounded(bar, 0u, err, polls);
}

// Sweep knobs (environment variables DSDPA_*), read once per process: the planner runs on every
// call and must not walk the environment there.
struct Knobs {
    int fwd_nw, fwd_nq, bwd_nw, bwd_nq;
    int gather_smem_kb, index_smem_kb, gather_qb, gather_threads, gather_nslab, bwd_two_pass;
};
static int env_int(const char* name, int fallback) {
    const char* s = std::getenv(name);
    if (!s || !*s) return fallback;
    return std::atoi(s);
}
static const Knobs& knobs() {
    static const Knobs k = {
        env_int("DSDPA_FWD_NW", 0), env_int("DSDPA_FWD_NQ", 0), env_int("DSDPA_BWD_NW", 0), env_int("DSDPA_BWD_NQ", 0),
        env_int("DSDPA_GATHER_SMEM_KB", 224), env_int("DSDPA_INDEX_SMEM_KB", 112), env_int("DSDPA_GATHER_QB", 0),
        env_int("DSDPA_GATHER_THREADS", 0), env_int("DSDPA_GATHER_NSLAB", 0), env_int("DSDPA_BWD_TWO_PASS", 1),
    };
    return k;
}

int validate_problem(const dsdpa_problem* p) {
    if (!p) return DSDPA_ERR_NULL_POINTER;
    if (p->dtype != DSDPA_F32 && p->dtype != DSDPA_BF16 && p->dtype != DSDPA_F16) return DSDPA_ERR_BAD_DTYPE;
    if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return DSDPA_ERR_BAD_HEAD_DIM;
    if (p->B <= 0 || p->V <= 0 || p->Hh <= 0 || p->W <= 0 || p->H <= 0 || p->S <= 0) return DSDPA_ERR_BAD_SHAPE;
    const unsigned known = DSDPA_FLAG_MAPS_FROM_L2 | DSDPA_FLAG_DETERMINISTIC | DSDPA_FLAG_SCATTER_GLOBAL |
                           DSDPA_FLAG_SCATTER | DSDPA_FLAG_ROUNDED_WEIGHTS;
    if (p->flags & ~known) return DSDPA_ERR_BAD_FLAGS;
    if ((p->flags & DSDPA_FLAG_DETERMINISTIC) && (p->flags & (DSDPA_FLAG_SCATTER | DSDPA_FLAG_SCATTER_GLOBAL)))
        return DSDPA_ERR_BAD_FLAGS;
    const long long L = (long long)p->W * p->H;
    // pixel offsets inside one map and the per-(batch, head) query index are 32-bit
    if (L * p->D * 4 >= (1ll << 31)) return DSDPA_ERR_BAD_SHAPE;
    if ((long long)p->V * L >= (1ll << 30)) return DSDPA_ERR_BAD_SHAPE;
    if ((long long)p->V * p->S >= (1ll << 30)) return DSDPA_ERR_BAD_SHAPE;
    if ((long long)p->B * p->Hh >= (1ll << 24)) return DSDPA_ERR_BAD_SHAPE;
    if (!(p->sm_scale == p->sm_scale)) return DSDPA_ERR_BAD_SHAPE;
    return DSDPA_OK;
}

TilePlan plan_tiles(const dsdpa_problem& p, bool backward, bool allow_priv) {
    const int L = p.W * p.H, VL = p.V * L;
    const long long map_bytes = (long long)L * p.D * dtype_size(p.dtype);
    const long long acc_bytes = (long long)L * p.D * 4;
    const RowGeom rg = row_geom(p.D, p.dtype);
    const int ch = (p.D * dtype_size(p.dtype) / 16) / rg.G;
    const int force_nw = backward ? knobs().bwd_nw : knobs().fwd_nw;
    const int force_nq = backward ? knobs().bwd_nq : knobs().fwd_nq;

    auto smem_need = [&](int nstage, int nw, bool priv) -> long long {
        return (long long)nstage * 2 * map_bytes + (priv ? 2 * acc_bytes : 0) + (long long)nw * kPlanRecBytesPerWarp + 32;
    };
    TilePlan best{};
    best.rounded_weights = !backward && (p.flags & DSDPA_FLAG_ROUNDED_WEIGHTS) && p.dtype != DSDPA_F32;
    // mbarrier transaction counts hold 2^20-1 bytes; each map completes on a barrier of its own
    const bool can_stage = !(p.flags & DSDPA_FLAG_MAPS_FROM_L2) && smem_need(1, 4, false) <= kPlanSmemMax &&
                           map_bytes < (1ll << 20);
    if (can_stage) {
        const bool want_priv = backward && allow_priv && !(p.flags & DSDPA_FLAG_SCATTER_GLOBAL) &&
                               smem_need(1, 8, true) <= kPlanSmemMax;
        double best_cost = 1e300;
        // forward: four samples per inner iteration leave registers for two query slots per group
        const int nqs_fwd[3] = { 2, 1, 1 }, nqs_bwd[2] = { 4, 1 };
        const int* nqs = backward ? nqs_bwd : nqs_fwd;
        const int n_nq = backward ? 2 : 3;
        for (int qi = 0; qi < n_nq; ++qi) {
            const int nq = nqs[qi];
            if (force_nq && nq != force_nq) continue;
            // multiples of four warps keep the four schedulers of an SM evenly loaded
            for (int nw = 16; nw >= 4; nw -= 4) {
                if (force_nw && nw != force_nw) continue;
                if (smem_need(1, nw, want_priv) > kPlanSmemMax) continue;
                const int nstage = smem_need(2, nw, want_priv) <= kPlanSmemMax ? 2 : 1;
                const int cap = nw * rg.NG * nq;
                const int tiles = (VL + cap - 1) / cap;
                const int qpt = (VL + tiles - 1) / tiles;
                const long long ctas = (long long)p.B * p.Hh * tiles;
                const int rounds = (qpt + nw * rg.NG - 1) / (nw * rg.NG);
                const long long waves = (ctas + kPlanSMs - 1) / kPlanSMs;
                // one warp step moves 8*CH 128-bit loads = 32*CH shared-memory wavefronts
                const double wf = 32.0 * ch * (backward ? 2.5 : 1.0);
                // a warp's step takes about a thousand cycles end to end (measured), so a CTA is
                // latency-bound until it has enough warps to cover that with wavefronts
                const double lat = backward ? 1200.0 : 1000.0;
                const double step = nw * wf > lat ? nw * wf : lat;
                const double stage_cost = nstage == 1 ? 2.0 * (double)map_bytes / 48.0 : 0.0;
                const double flush_cost = want_priv ? 2.0 * (double)acc_bytes / 32.0 : 0.0;
                const double cta_time = p.V * ((double)rounds * p.S * step + stage_cost + flush_cost + 2000.0);
                const double cost = (double)waves * cta_time;
                if (cost < best_cost) {
                    best_cost = cost;
                    best.staged = true;
                    best.priv = want_priv;
                    best.nstage = nstage;
                    best.nw = nw;
                    best.nq = nq;
                    best.tiles = tiles;
                    best.q_per_tile = qpt;
                    best.smem = (size_t)smem_need(nstage, nw, want_priv);
                    best.ctas = ctas;
                }
            }
        }
        if (best.staged) return best;
    }
    // maps served from L2/L1: one query per group, many small CTAs
    int nw = force_nw ? force_nw : 8;
    if (nw * 32 > 256) nw = 8;
    best.staged = false;
    best.priv = false;
    best.nstage = 0;
    best.nw = nw;
    best.nq = 1;
    const int cap = nw * rg.NG;
    best.tiles = (VL + cap - 1) / cap;
    best.q_per_tile = cap;
    best.smem = (size_t)nw * kPlanRecBytesPerWarp + 32;
    best.ctas = (long long)p.B * p.Hh * best.tiles;
    return best;
}

GatherPlan plan_gather(const dsdpa_problem& p) {
    GatherPlan g{};
    const int L = p.W * p.H;
    const long long A = (long long)p.H * (p.W + 1);   // anchors: pixel pairs (x-1, x) of one map row
    const long long rowb = (long long)p.D * dtype_size(p.dtype);
    const long long per_query = 2 * rowb + (long long)p.S * 8;
    g.gather_threads = knobs().gather_threads;
    if (g.gather_threads < 32 || g.gather_threads > gather_max_threads(p.dtype) || g.gather_threads % 32)
        g.gather_threads = gather_max_threads(p.dtype);
    // every group of lanes keeps a small ring of index entries in shared memory
    const RowGeom rg = row_geom(p.D, p.dtype);
    const long long chunk = rg.G < 8 ? rg.G : 8;
    const long long ring_bytes = (long long)(g.gather_threads / 32) * rg.NG * (2 * chunk * 16 + 16);
    const long long budget = (long long)knobs().gather_smem_kb * 1024;
    long long qb_max = ((budget < kPlanSmemMax ? budget : kPlanSmemMax) - 64 - ring_bytes) / per_query;
    qb_max &= ~1ll;  // even, so that every tile's scalars start on a 16-byte boundary
    // entries hold byte offsets into the tile's rows and scalars as 32-bit fields; one segment's
    // entry count must stay an int
    while (qb_max > 2 && qb_max * p.S * 2 > (1ll << 30)) qb_max -= 2;
    // The index builder keeps one histogram over the anchors per sample-taking warp: one per warp
    // when they fit, fewer for large maps (slower to build, same lists).
    // (beside the histograms: the lists' first entries [A], a partial sum per thread, the length buckets)
    const long long fixed_ints = kIndexWarpsDefault * 32 + (long long)kMaxSlabs * kLenBuckets;
    long long nhist = ((long long)kPlanSmemMax / 4 - 16 - fixed_ints) / A - 1;
    if (nhist > kIndexWarpsDefault) nhist = kIndexWarpsDefault;
    if (qb_max < 2 || nhist < 1 || A + 1 >= (1ll << 30)) return g;  // ok = false
    size_t index_smem = (size_t)((nhist + 1) * A + fixed_ints) * sizeof(int);
    {
        // The index builder scatters 16-byte entries; with many CTAs per SM their half-written
        // 32-byte sectors outgrow L2 and are evicted before they are complete.  Asking for more
        // shared memory than needed caps the CTAs per SM at two (measured best).
        const size_t floor_kb = (size_t)knobs().index_smem_kb;
        if (floor_kb * 1024 > index_smem && floor_kb * 1024 <= (size_t)kPlanSmemMax) index_smem = floor_kb * 1024;
    }
    const int force_qb = knobs().gather_qb;
    if (force_qb >= 2 && force_qb <= qb_max) qb_max = force_qb & ~1;
    g.tpv = (int)((L + qb_max - 1) / qb_max);
    int qb = (L + g.tpv - 1) / g.tpv;
    qb += qb & 1;
    g.QB = qb;
    g.ok = true;
    g.A = (int)A;
    g.nhist = (int)nhist;
    g.gather_smem = (size_t)qb * 2 * rowb + (((size_t)qb * p.S * 8 + 15) & ~(size_t)15) + 16 + (size_t)ring_bytes;
    // One CTA per SM: when the grid is only a few waves long and the last one is poorly filled,
    // split every unit's map rows over 2-4 CTAs.
    {
        const long long units = (long long)p.B * p.Hh * p.V;
        int best = 1;
        double best_eff = 0.0;
        for (int ns = 1; ns <= kMaxSlabs && ns <= p.H; ++ns) {
            const long long ctas = units * ns;
            const long long waves = (ctas + kPlanSMs - 1) / kPlanSMs;
            // every extra CTA of a unit reloads the tiles (2% per split), and the slabs are whole
            // map rows, so the largest slab sets the pace
            const int rows = (p.H + ns - 1) / ns;
            const double eff = (double)ctas / (double)(waves * kPlanSMs) * (1.0 - 0.02 * (ns - 1)) *
                               ((double)p.H / ((double)rows * ns));
            if (eff > best_eff + 1e-9) { best_eff = eff; best = ns; }
        }
        const int force = knobs().gather_nslab;
        g.nslab = force >= 1 && force <= kMaxSlabs && force <= p.H ? force : best;
        g.gather_ctas = units * g.nslab;
    }
    const long long T = (long long)p.V * g.tpv;
    g.segments = (long long)p.B * T * p.V;
    g.index_smem = index_smem;
    g.scal_bytes = (((size_t)p.B * p.Hh * T * p.V * qb * p.S * 8) + 16 + 255) & ~(size_t)255;
    g.seg_entries = (int)((long long)qb * p.S * 2);
    g.entries_bytes = (((size_t)g.segments * g.seg_entries * 16) + 255) & ~(size_t)255;
    g.sched_bytes = (((size_t)g.segments * A * 16) + 255) & ~(size_t)255;
    g.hdr_bytes = (((size_t)g.segments * g.nslab * 8) + 255) & ~(size_t)255;
    return g;
}

// Which backward form a problem runs with.
static bool use_two_pass(const dsdpa_problem& p, const GatherPlan& g) {
    if (!g.ok) return false;
    if (p.flags & (DSDPA_FLAG_SCATTER | DSDPA_FLAG_SCATTER_GLOBAL)) return false;
    if (p.flags & DSDPA_FLAG_DETERMINISTIC) return true;
    return knobs().bwd_two_pass != 0;
}

static bool misaligned(const void* p) { return ((uintptr_t)p & 15u) != 0; }

struct DeviceGuard {
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) (void)cudaSetDevice(prev);
    }
};

// A mirror may lie in another GPU's memory: kernels launched on `device` (the current device)
// must be allowed to store to it, or the first store faults.  Looked up once per pair of devices.
static int ensure_mirror_access(const void* ptr, int device) {
    if (!ptr) return DSDPA_OK;
    cudaPointerAttributes attr{};
    cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
    if (e != cudaSuccess) return cuda_fail(e);
    if (attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeManaged) return DSDPA_OK;
    if (attr.type != cudaMemoryTypeDevice) return DSDPA_ERR_PEER_ACCESS;  // not known to CUDA at all
    const int owner = attr.device;
    if (owner == device) return DSDPA_OK;
    static std::atomic<unsigned char> enabled[64][64];
    const bool cacheable = device >= 0 && device < 64 && owner >= 0 && owner < 64;
    if (cacheable && enabled[device][owner].load()) return DSDPA_OK;
    int can = 0;
    if ((e = cudaDeviceCanAccessPeer(&can, device, owner)) != cudaSuccess) return cuda_fail(e);
    if (!can) return DSDPA_ERR_PEER_ACCESS;
    e = cudaDeviceEnablePeerAccess(owner, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();  // not an error: somebody else switched it on
        e = cudaSuccess;
    }
    if (e != cudaSuccess) return cuda_fail(e);
    if (cacheable) enabled[device][owner].store(1);
    return DSDPA_OK;
}

static cudaError_t error_word_ptr(int device, int** out) {
    static int* cache[64] = {};
    if (device >= 0 && device < 64 && cache[device]) {
        *out = cache[device];
        return cudaSuccess;
    }
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_error_word);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) cache[device] = (int*)ptr;
    *out = (int*)ptr;
    return cudaSuccess;
}

// ---- copy of a finished result to its mirror (scatter forms of the backward only) ---
__global__ void __launch_bounds__(512) copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        stg128(dst + i, ldg128_stream(src + i));
}
static cudaError_t launch_copy16(const void* src, void* dst, size_t bytes, cudaStream_t s) {
    const size_t n16 = bytes / 16;  // results are whole 16-byte rows
    if (n16 == 0) return cudaSuccess;
    const size_t want = (n16 + 511) / 512;
    const unsigned grid = (unsigned)(want < (size_t)kPlanSMs * 4 ? want : (size_t)kPlanSMs * 4);
    copy16_kernel<<<grid, 512, 0, s>>>((const uint4*)src, (uint4*)dst, n16);
    return cudaGetLastError();
}

}  // namespace dsdpa

using namespace dsdpa;

extern "C" {

const char* dsdpa_status_string(int status) {
    switch (status) {
        case DSDPA_OK: return "ok";
        case DSDPA_ERR_NULL_POINTER: return "null pointer";
        case DSDPA_ERR_BAD_DTYPE: return "unsupported dtype (float32, bfloat16 and float16 are supported)";
        case DSDPA_ERR_BAD_HEAD_DIM: return "head dimension must be one of 16, 32, 64, 128, 256";
        case DSDPA_ERR_BAD_SHAPE: return "bad shape (non-positive extent or too large)";
        case DSDPA_ERR_MISALIGNED: return "pointer is not 16-byte aligned";
        case DSDPA_ERR_WORKSPACE: return "workspace missing or too small";
        case DSDPA_ERR_BAD_FLAGS: return "unknown or contradictory flags";
        case DSDPA_ERR_CUDA: return "CUDA runtime error";
        case DSDPA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
        case DSDPA_ERR_TOO_LARGE: return "problem exceeds the maximum of this entry point";
        case DSDPA_ERR_PEER_ACCESS: return "a mirror lies in memory the launching device cannot store to";
        case DSDPA_ERR_DEVICE_BOUNDS: return "a kernel of the checked build computed an index out of range (access skipped)";
        default: return "unknown status";
    }
}

int dsdpa_version(void) { return DSDPA_VERSION; }

int dsdpa_last_cuda_error(void) { return t_last_cuda_error; }

unsigned long long dsdpa_kernel_launches(void) { return g_launches.load(); }

int dsdpa_describe_plan(const dsdpa_problem* p, char* text, size_t cap) {
    int st = validate_problem(p);
    if (st != DSDPA_OK) return st;
    if (!text || cap == 0) return DSDPA_ERR_NULL_POINTER;
    const GatherPlan g = plan_gather(*p);
    const bool two = use_two_pass(*p, g);
    const TilePlan f = plan_tiles(*p, false, false), b = plan_tiles(*p, true, !two);
    char tail[160] = "";
    if (two)
        std::snprintf(tail, sizeof tail, " bwd_gather[tpv=%d QB=%d nslab=%d ctas=%lld smem=%zu segments=%lld]", g.tpv, g.QB,
                      g.nslab, g.gather_ctas, g.gather_smem, g.segments);
    std::snprintf(text, cap,
                  "fwd[%s nstage=%d nw=%d nq=%d tiles=%d q_per_tile=%d ctas=%lld smem=%zu] "
                  "bwd_%s[%s%s nstage=%d nw=%d nq=%d tiles=%d q_per_tile=%d ctas=%lld smem=%zu]%s",
                  f.staged ? (f.rounded_weights ? "staged+rw" : "staged") : (f.rounded_weights ? "l2+rw" : "l2"), f.nstage,
                  f.nw, f.nq, f.tiles, f.q_per_tile, f.ctas, f.smem,
                  two ? "pass_a" : "scatter", b.staged ? "staged" : "l2", b.priv ? "+priv" : "", b.nstage, b.nw, b.nq,
                  b.tiles, b.q_per_tile, b.ctas, b.smem, tail);
    return DSDPA_OK;
}

int dsdpa_forward(const dsdpa_problem* p, const void* q, const void* k, const void* v, const float* coords,
                  void* out, float* lse, int device, void* stream) {
    return dsdpa_forward_mirrored(p, q, k, v, coords, out, lse, nullptr, device, stream);
}

int dsdpa_forward_mirrored(const dsdpa_problem* p, const void* q, const void* k, const void* v, const float* coords,
                           void* out, float* lse, void* out_mirror, int device, void* stream) {
    int st = validate_problem(p);
    if (st != DSDPA_OK) return st;
    if (!q || !k || !v || !coords || !out || !lse) return DSDPA_ERR_NULL_POINTER;
    if (misaligned(q) || misaligned(k) || misaligned(v) || misaligned(coords) || misaligned(out) || misaligned(lse) ||
        misaligned(out_mirror))
        return DSDPA_ERR_MISALIGNED;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    if ((st = ensure_mirror_access(out_mirror, device)) != DSDPA_OK) return st;
    int* err_word = nullptr;
    cudaError_t e = error_word_ptr(device, &err_word);
    if (e != cudaSuccess) return cuda_fail(e);

    const TilePlan plan = plan_tiles(*p, false, false);
    FwdParams fp{};
    fp.q = q; fp.k = k; fp.v = v; fp.coords = coords; fp.out = out; fp.out_mirror = out_mirror; fp.lse = lse;
    fp.B = p->B; fp.V = p->V; fp.Hh = p->Hh; fp.W = p->W; fp.H = p->H; fp.L = p->W * p->H; fp.S = p->S;
    fp.scale2 = p->sm_scale * kLog2e;
    fp.hw = (float)(p->W - 1) * 0.5f;
    fp.hh = (float)(p->H - 1) * 0.5f;
    fp.tiles = plan.tiles;
    fp.q_per_tile = plan.q_per_tile;
    fp.nstage = plan.nstage;
    fp.map_bytes = (unsigned)((size_t)fp.L * p->D * dtype_size(p->dtype));
    fp.err = err_word;
    cudaStream_t s = (cudaStream_t)stream;
    switch (p->dtype) {
        case DSDPA_F32: e = launch_forward<float>(fp, plan, p->D, s); break;
        case DSDPA_BF16: e = launch_forward<__nv_bfloat16>(fp, plan, p->D, s); break;
        default: e = launch_forward<__half>(fp, plan, p->D, s); break;
    }
    if (e != cudaSuccess) return cuda_fail(e);
    g_launches += 1;
    return DSDPA_OK;
}

// fp32 dK/dV accumulators inside the workspace.  Scatter forms: one pair of maps for 16-bit
// storage (fp32 storage accumulates in dk/dv).  Two-pass form: a "left" and a "right" pair;
// for fp32 storage the left pair is dk/dv themselves.
static size_t accumulator_bytes(const dsdpa_problem& p, bool two_pass) {
    const size_t n = (size_t)p.B * p.V * p.Hh * p.W * p.H * p.D;
    const size_t maps = (p.dtype == DSDPA_F32 ? 0 : 2) + (two_pass ? 2 : 0);
    return maps == 0 ? 0 : ((maps * n * sizeof(float) + 255) & ~(size_t)255);
}

size_t dsdpa_backward_workspace_bytes(const dsdpa_problem* p) {
    if (validate_problem(p) != DSDPA_OK) return 0;
    const GatherPlan g = plan_gather(*p);
    const bool two = use_two_pass(*p, g);
    size_t bytes = accumulator_bytes(*p, two);
    if (two) bytes += g.scal_bytes + g.entries_bytes + g.sched_bytes + g.hdr_bytes;
    return bytes;
}

int dsdpa_backward_supports_dcoords(const dsdpa_problem* p) {
    if (validate_problem(p) != DSDPA_OK) return 0;
    return use_two_pass(*p, plan_gather(*p)) ? 1 : 0;
}

int dsdpa_backward(const dsdpa_problem* p, const void* q, const void* k, const void* v, const float* coords,
                   const void* out, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                   float* dcoords, void* workspace, size_t workspace_bytes, int device, void* stream) {
    return dsdpa_backward_mirrored(p, q, k, v, coords, out, lse, dout, dq, dk, dv, dcoords, workspace, workspace_bytes,
                                   nullptr, device, stream);
}

int dsdpa_backward_mirrored(const dsdpa_problem* p, const void* q, const void* k, const void* v, const float* coords,
                            const void* out, const float* lse, const void* dout, void* dq, void* dk, void* dv,
                            float* dcoords, void* workspace, size_t workspace_bytes, const dsdpa_mirrors* mirrors,
                            int device, void* stream) {
    const dsdpa_mirrors mir = mirrors ? *mirrors : dsdpa_mirrors{ nullptr, nullptr, nullptr, nullptr };
    if (misaligned(mir.out) || misaligned(mir.dq) || misaligned(mir.dk) || misaligned(mir.dv)) return DSDPA_ERR_MISALIGNED;
    int st = validate_problem(p);
    if (st != DSDPA_OK) return st;
    if (!q || !k || !v || !coords || !out || !lse || !dout || !dq || !dk || !dv) return DSDPA_ERR_NULL_POINTER;
    if (misaligned(q) || misaligned(k) || misaligned(v) || misaligned(coords) || misaligned(out) || misaligned(lse) ||
        misaligned(dout) || misaligned(dq) || misaligned(dk) || misaligned(dv) || misaligned(workspace) ||
        misaligned(dcoords))
        return DSDPA_ERR_MISALIGNED;
    const size_t need = dsdpa_backward_workspace_bytes(p);
    if (need > 0 && (!workspace || workspace_bytes < need)) return DSDPA_ERR_WORKSPACE;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    for (const void* m : { mir.out, mir.dq, mir.dk, mir.dv })
        if ((st = ensure_mirror_access(m, device)) != DSDPA_OK) return st;
    int* err_word = nullptr;
    cudaError_t e = error_word_ptr(device, &err_word);
    if (e != cudaSuccess) return cuda_fail(e);
    cudaStream_t s = (cudaStream_t)stream;

    const GatherPlan gp = plan_gather(*p);
    const bool two_pass = use_two_pass(*p, gp);
    // the coordinate gradient is computed by the two-pass form's first pass only
    if (dcoords && !two_pass) return DSDPA_ERR_BAD_FLAGS;
    const size_t n = (size_t)p->B * p->V * p->Hh * p->W * p->H * p->D;
    if (dcoords) {
        const size_t nc = (size_t)p->B * p->V * p->W * p->H * p->V * p->S * 2;
        if ((e = cudaMemsetAsync(dcoords, 0, nc * sizeof(float), s)) != cudaSuccess) return cuda_fail(e);
    }
    const size_t acc_bytes = accumulator_bytes(*p, two_pass);
    float* dk32 = p->dtype == DSDPA_F32 ? (float*)dk : (float*)workspace;
    float* dv32 = p->dtype == DSDPA_F32 ? (float*)dv : (float*)workspace + n;
    // two-pass form: the second ("right") pair of maps lies behind the first in the workspace
    float* dk_right = two_pass ? (float*)workspace + (p->dtype == DSDPA_F32 ? 0 : 2 * n) : nullptr;
    float* dv_right = two_pass ? dk_right + n : nullptr;
    if (p->dtype == DSDPA_F32) {
        if ((e = cudaMemsetAsync(dk32, 0, n * sizeof(float), s)) != cudaSuccess) return cuda_fail(e);
        if ((e = cudaMemsetAsync(dv32, 0, n * sizeof(float), s)) != cudaSuccess) return cuda_fail(e);
    }
    if (acc_bytes > 0 && (e = cudaMemsetAsync(workspace, 0, acc_bytes, s)) != cudaSuccess) return cuda_fail(e);

    const int L = p->W * p->H;
    const float hw = (float)(p->W - 1) * 0.5f, hh = (float)(p->H - 1) * 0.5f;
    char* ws = (char*)workspace + acc_bytes;
    float2* scal = two_pass ? (float2*)ws : nullptr;
    uint4* entries = two_pass ? (uint4*)(ws + gp.scal_bytes) : nullptr;
    int4* sched = two_pass ? (int4*)(ws + gp.scal_bytes + gp.entries_bytes) : nullptr;
    int2* sched_hdr = two_pass ? (int2*)(ws + gp.scal_bytes + gp.entries_bytes + gp.sched_bytes) : nullptr;

    if (two_pass) {
        // pixel-sorted sample lists, shared by all heads
        IndexParams ip{};
        ip.coords = coords; ip.sched = sched; ip.sched_hdr = sched_hdr; ip.entries = entries;
        ip.B = p->B; ip.V = p->V; ip.W = p->W; ip.H = p->H; ip.L = L; ip.S = p->S;
        ip.hw = hw; ip.hh = hh; ip.tpv = gp.tpv; ip.QB = gp.QB;
        ip.rowb = p->D * dtype_size(p->dtype); ip.seg_entries = gp.seg_entries;
        ip.A = gp.A; ip.nhist = gp.nhist; ip.nslab = gp.nslab; ip.err = err_word;
        static bool index_attr[64] = {};
        if ((e = detail::allow_big_smem(index_build_kernel<kIndexWarpsDefault>, index_attr)) != cudaSuccess) return cuda_fail(e);
        index_build_kernel<kIndexWarpsDefault><<<(unsigned)gp.segments, kIndexWarpsDefault * 32, gp.index_smem, s>>>(ip);
        if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
        g_launches += 1;
    }

    const TilePlan plan = plan_tiles(*p, true, !two_pass);
    BwdParams bp{};
    bp.q = q; bp.k = k; bp.v = v; bp.coords = coords; bp.out = out; bp.lse = lse; bp.dout = dout;
    bp.dq = dq; bp.out_mirror = mir.out; bp.dq_mirror = mir.dq; bp.dk32 = dk32; bp.dv32 = dv32; bp.dcoords = dcoords;
    bp.B = p->B; bp.V = p->V; bp.Hh = p->Hh; bp.W = p->W; bp.H = p->H; bp.L = L; bp.S = p->S;
    bp.sm_scale = p->sm_scale;
    bp.scale2 = p->sm_scale * kLog2e;
    bp.hw = hw;
    bp.hh = hh;
    bp.tiles = plan.tiles;
    bp.q_per_tile = plan.q_per_tile;
    bp.nstage = plan.nstage;
    bp.map_bytes = (unsigned)((size_t)L * p->D * dtype_size(p->dtype));
    bp.acc_bytes = (unsigned)((size_t)L * p->D * 4);
    bp.err = err_word;
    bp.scal = scal;
    bp.tpv = gp.tpv;
    bp.QB = gp.QB;
    switch (p->dtype) {
        case DSDPA_F32: e = launch_backward_main<float>(bp, plan, p->D, two_pass, dcoords != nullptr, s); break;
        case DSDPA_BF16: e = launch_backward_main<__nv_bfloat16>(bp, plan, p->D, two_pass, dcoords != nullptr, s); break;
        default: e = launch_backward_main<__half>(bp, plan, p->D, two_pass, dcoords != nullptr, s); break;
    }
    if (e != cudaSuccess) return cuda_fail(e);
    g_launches += 1;

    if (two_pass) {
        GatherParams g{};
        g.q = q; g.dout = dout; g.scal = scal; g.sched = sched; g.sched_hdr = sched_hdr; g.entries = entries;
        g.dk_left = dk32; g.dv_left = dv32; g.dk_right = dk_right; g.dv_right = dv_right;
        g.dk = dk; g.dv = dv; g.dk_mirror = mir.dk; g.dv_mirror = mir.dv;
        g.B = p->B; g.V = p->V; g.Hh = p->Hh; g.W = p->W; g.H = p->H; g.L = L; g.S = p->S; g.tpv = gp.tpv; g.QB = gp.QB;
        g.seg_entries = gp.seg_entries; g.A = gp.A;
        g.nslab = gp.nslab;
        g.err = err_word;
        switch (p->dtype) {
            case DSDPA_F32: e = launch_backward_gather<float>(g, gp, p->D, s); break;
            case DSDPA_BF16: e = launch_backward_gather<__nv_bfloat16>(g, gp, p->D, s); break;
            default: e = launch_backward_gather<__half>(g, gp, p->D, s); break;
        }
        if (e != cudaSuccess) return cuda_fail(e);
        g_launches += 1;
    }

    // the gather pass hands the finished maps over itself; the scatter forms need a pass of
    // their own for the rounding to the storage type and for the mirrors
    if (!two_pass) {
        if (p->dtype == DSDPA_BF16) {
            if ((e = launch_cast_from_f32<__nv_bfloat16>(dk32, dk, n, s)) != cudaSuccess) return cuda_fail(e);
            if ((e = launch_cast_from_f32<__nv_bfloat16>(dv32, dv, n, s)) != cudaSuccess) return cuda_fail(e);
            g_launches += 2;
        } else if (p->dtype == DSDPA_F16) {
            if ((e = launch_cast_from_f32<__half>(dk32, dk, n, s)) != cudaSuccess) return cuda_fail(e);
            if ((e = launch_cast_from_f32<__half>(dv32, dv, n, s)) != cudaSuccess) return cuda_fail(e);
            g_launches += 2;
        }
        const size_t bytes = n * dtype_size(p->dtype);
        if (mir.dk) {
            if ((e = launch_copy16(dk, mir.dk, bytes, s)) != cudaSuccess) return cuda_fail(e);
            g_launches += 1;
        }
        if (mir.dv) {
            if ((e = launch_copy16(dv, mir.dv, bytes, s)) != cudaSuccess) return cuda_fail(e);
            g_launches += 1;
        }
    }
    return DSDPA_OK;
}

int dsdpa_peer_export(const void* ptr, int device, unsigned char handle[DSDPA_PEER_HANDLE_BYTES], size_t* offset) {
    static_assert(sizeof(cudaIpcMemHandle_t) == DSDPA_PEER_HANDLE_BYTES, "handle size");
    if (!ptr || !handle || !offset) return DSDPA_ERR_NULL_POINTER;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    // start of the allocation that holds ptr: a driver call, reached through the runtime
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found;
    cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &found);
    if (e != cudaSuccess) return cuda_fail(e);
    if (!fn || found != cudaDriverEntryPointSuccess) return cuda_fail(cudaErrorNotSupported);
    unsigned long long base = 0;
    size_t size = 0;
    if (((range_fn)fn)(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0) return cuda_fail(cudaErrorInvalidValue);
    cudaIpcMemHandle_t h;
    if ((e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base)) != cudaSuccess) return cuda_fail(e);
    std::memcpy(handle, &h, sizeof h);
    *offset = (size_t)((uintptr_t)ptr - (uintptr_t)base);
    return DSDPA_OK;
}

int dsdpa_peer_import(const unsigned char handle[DSDPA_PEER_HANDLE_BYTES], size_t offset, int device, void** ptr) {
    if (!handle || !ptr) return DSDPA_ERR_NULL_POINTER;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof h);
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e);
    *ptr = (char*)base + offset;
    return DSDPA_OK;
}

int dsdpa_peer_release(void* ptr, size_t offset, int device) {
    if (!ptr) return DSDPA_ERR_NULL_POINTER;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    cudaError_t e = cudaIpcCloseMemHandle((char*)ptr - offset);
    return e == cudaSuccess ? DSDPA_OK : cuda_fail(e);
}

int dsdpa_device_error(int device) {
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e);
    int word = 0;
    if ((e = cudaMemcpyFromSymbol(&word, g_error_word, sizeof(int))) != cudaSuccess) return cuda_fail(e);
    if (word == 0) return DSDPA_OK;
    const int zero = 0;
    if ((e = cudaMemcpyToSymbol(g_error_word, &zero, sizeof(int))) != cudaSuccess) return cuda_fail(e);
    return word == kErrBounds ? DSDPA_ERR_DEVICE_BOUNDS : DSDPA_ERR_DEVICE_TIMEOUT;
}

int dsdpa_selftest_bounded_wait(unsigned polls, int device, void* stream) {
    if (polls == 0 || polls > (1u << 20)) return DSDPA_ERR_BAD_SHAPE;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err);
    int* err_word = nullptr;
    cudaError_t e = error_word_ptr(device, &err_word);
    if (e != cudaSuccess) return cuda_fail(e);
    selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(polls, err_word);
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
    g_launches += 1;
    return DSDPA_OK;
}

int dsdpa_build_is_checked(void) { return kBoundsCheck ? 1 : 0; }

}  // extern "C"
