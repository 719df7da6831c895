// C ABI of the sweep: argument checks, workspace carving and the launch schedule.
#include <math.h>

#include "g2d_common.cuh"

#include <mutex>
#include <vector>

namespace g2d {
std::atomic<unsigned long long> g_launches{0};
}

using namespace g2d;

namespace {

// Optional per-launch timing of the fused sweep (profiling entry point only): one event pair per launch.
struct LaunchTimer {
    struct Item { cudaEvent_t begin, end; int kind; };
    std::vector<Item> items;
    cudaStream_t stream;
    bool ok = true;
    void begin_on(int kind, cudaStream_t on) {  // a launch on another stream than the previous one (the null stream included)
        stream = on;
        begin(kind);
    }
    void begin(int kind) {
        Item it{};
        it.kind = kind;
        ok = ok && cudaEventCreate(&it.begin) == cudaSuccess && cudaEventCreate(&it.end) == cudaSuccess;
        if (ok) ok = cudaEventRecord(it.begin, stream) == cudaSuccess;
        items.push_back(it);
    }
    void end() {
        if (ok && !items.empty()) ok = cudaEventRecord(items.back().end, stream) == cudaSuccess;
    }
};

// Algorithmic multiply-adds (x2 = flops) of one band update in tile mode: exact, no padding counted.
double band_flops(int64_t m, int64_t n, int64_t s0, int64_t s1, int64_t s_end, int64_t T = TILE) {
    const int64_t TILE = T;
    const int64_t nI = ceil_div(m, TILE), nJ = ceil_div(n, TILE);
    double flops = 0;
    for (int64_t TI = 0; TI < nI; ++TI)
        for (int64_t TJ = 0; TJ < nJ; ++TJ) {
            if (TI + TJ < s1 || TI + TJ >= s_end) continue;
            const double rows = (double)(TI == nI - 1 ? m - TI * TILE : TILE), cols = (double)(TJ == nJ - 1 ? n - TJ * TILE : TILE);
            int64_t lo = s0 - TJ, hi = s1 - TJ;
            lo = lo < 0 ? 0 : lo; hi = hi > TI ? TI : hi;
            if (hi > lo) flops += 2.0 * rows * cols * (double)((hi - lo) * TILE);
            lo = s0 - TI; hi = s1 - TI;
            lo = lo < 0 ? 0 : lo; hi = hi > TJ ? TJ : hi;
            if (hi > lo) flops += 2.0 * rows * cols * (double)((hi - lo) * TILE);
        }
    return flops;
}

// Last launch of a sweep that used the tensor-core update kernels.  Their waits on hardware barriers are bounded; a
// wait that ran out made its CTA skip its additions and set `flag`.  Such a result must not pass for a valid one:
// the whole output is overwritten with NaN and the caller's status word (if any) is set to -1.  Costs one load per
// thread when all went well.
__global__ void sweep_finish_kernel(const int *__restrict__ flag, int32_t *status, float *y, int64_t count) {
    if (*flag == 0) return;
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(status, -1);
    const float poison = __int_as_float(0x7fc00000);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (int64_t)gridDim.x * blockDim.x) y[t] = poison;
}
int launch_sweep_finish(const int *flag, int32_t *status, float *y, int64_t count, cudaStream_t stream) {
    sweep_finish_kernel<<<148, 256, 0, stream>>>(flag, status, y, count);
    return check_launch();
}

constexpr int kDefaultOuterTiles = 8;  // tile anti-diagonals gathered into one far update (512 stages)

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// The tensor-core macro updates serve one float matrix whose rows are 16-byte multiples (a TMA requirement).
inline bool tc_eligible(const g2d_sweep_desc *d) {
    return d->dtype == G2D_F32 && d->batch == 1 && d->m % 4 == 0 && d->n % 4 == 0 && d->reserved != 1;
}
inline size_t tc_extra_bytes(const g2d_sweep_desc *d) {
    const size_t mn = align256(4 * (size_t)d->m * d->n), mm = align256(4 * (size_t)d->m * d->m), nn = align256(4 * (size_t)d->n * d->n);
    return 256 + 4 * mn + 2 * mm + 2 * nn + 4 * mn;  // flag, E^T and C splits, L and U^T splits, far and neighbour planes of the pipelined schedule
}

int check_sweep(const g2d_sweep_desc *d) {
    if (!d) return G2D_ERR_BAD_ARGUMENT;
    if (d->dtype != G2D_F32 && d->dtype != G2D_F64) return G2D_ERR_BAD_ARGUMENT;
    if (d->batch < 0 || d->m < 0 || d->n < 0) return G2D_ERR_BAD_ARGUMENT;
    if (d->quant_kind != G2D_Q_ROUND && d->quant_kind != G2D_Q_AFFINE && d->quant_kind != G2D_Q_FORCED) return G2D_ERR_UNSUPPORTED;
    if (d->outer_tiles < 0) return G2D_ERR_BAD_ARGUMENT;
    return G2D_OK;
}

// Feedback between macro tiles: on the tensor cores when the operand planes exist, else the general FFMA update.
template <typename F>
int launch_macro_update(const BandArgs<F> &bm, const TcPlanes *planes, const MacroTcMaps *maps, cudaStream_t stream) {
    if (planes != nullptr) {
        if constexpr (sizeof(F) == sizeof(float))
            return launch_macro_update_tc(maps, *planes, (float *)bm.y, (float *)bm.c, bm.m, bm.n, (int)bm.s0, (int)bm.s1, (int)bm.s_end, stream);
    }
    return launch_band_update<F>(bm, stream);
}

constexpr int MACRO = 2 * TILE;          // macro tile edge: 2 x 2 tiles
constexpr int kDefaultOuterMacro = 4;    // macro anti-diagonals per far update (512 stages)

// Macro schedule: the matrix is cut into 128 x 128 macro tiles of 2 x 2 tiles.  A macro anti-diagonal W is swept in
// three tile launches (its even-even tiles, then the mixed ones, then the odd-odd ones) with the feedback inside each
// macro tile applied by two small tile-level updates; feedback between macro tiles is rank-128 per macro anti-diagonal
// (near update, into the rest of the group) and rank-512 per group (far update), so that every operand block of
// those updates is a whole 128 x 128 block.
template <typename F>
int sweep_macro(const g2d_sweep_desc *d, SweepArgs<F> &a, BandArgs<F> &b64, cudaStream_t stream, LaunchTimer *timer, double *flops,
                const TcPlanes *planes) {
    MacroTcMaps maps;
    if (planes != nullptr) {
        const int status = macro_tc_prepare(&maps, *planes, d->m, d->n);
        if (status != G2D_OK) return status;
    }
    const int nI2 = (int)ceil_div(d->m, MACRO), nJ2 = (int)ceil_div(d->n, MACRO);
    const int waves = nI2 + nJ2 - 1;
    const int outer = d->outer_tiles > 0 ? (d->outer_tiles + 1) / 2 : kDefaultOuterMacro;
    BandArgs<F> bm = b64;
    bm.P = MACRO; bm.Q = MACRO; bm.mode = BAND_GENERAL; bm.filter = 0;
    auto timed = [&](int kind, auto &&launch) {
        if (timer) timer->begin(kind);
        const int status = launch();
        if (timer) timer->end();
        return status;
    };
    for (int W0 = 0; W0 < waves; W0 += outer) {
        const int W1 = W0 + outer < waves ? W0 + outer : waves;
        for (int W = W0; W < W1; ++W) {
            int status = timed(0, [&] { return launch_tile_sweep<F>(a, 2 * W, stream, 1); });
            if (status != G2D_OK) return status;
            b64.s0 = 2 * W; b64.s1 = 2 * W + 1; b64.s_end = 2 * W + 2; b64.filter = 1;
            status = timed(1, [&] { return launch_band_update<F>(b64, stream); });
            if (status != G2D_OK) return status;
            status = timed(0, [&] { return launch_tile_sweep<F>(a, 2 * W + 1, stream, 0); });
            if (status != G2D_OK) return status;
            b64.s0 = 2 * W + 1; b64.s1 = 2 * W + 2; b64.s_end = 2 * W + 3; b64.filter = 2;
            status = timed(1, [&] { return launch_band_update<F>(b64, stream); });
            if (status != G2D_OK) return status;
            status = timed(0, [&] { return launch_tile_sweep<F>(a, 2 * W + 2, stream, 2); });
            if (status != G2D_OK) return status;
            if (W + 1 < W1) {
                bm.s0 = W; bm.s1 = W + 1; bm.s_end = W1;
                status = timed(1, [&] { return launch_macro_update<F>(bm, planes, &maps, stream); });
                if (flops) flops[1] += band_flops(d->m, d->n, bm.s0, bm.s1, bm.s_end, MACRO) * (double)d->batch;
                if (status != G2D_OK) return status;
            }
        }
        if (W1 < waves) {
            bm.s0 = W0; bm.s1 = W1; bm.s_end = waves;
            const int status = timed(2, [&] { return launch_macro_update<F>(bm, planes, &maps, stream); });
            if (flops) flops[2] += band_flops(d->m, d->n, bm.s0, bm.s1, bm.s_end, MACRO) * (double)d->batch;
            if (status != G2D_OK) return status;
        }
    }
    return G2D_OK;
}

// Side streams and events of the pipelined schedule.  A device has four lanes; calls take them round robin and hold a
// lane's lock while they enqueue, so sweeps that a caller runs concurrently on several streams (or from several host
// threads) never interleave their event records on one lane.  All four lanes of a device are built by the first
// pipelined call on it, which therefore must not run inside a stream capture (stream and event creation is not
// capturable): during capture, a device whose lanes do not exist yet gets G2D_ERR_UNSUPPORTED.
struct PipeLane {
    cudaStream_t tiles = nullptr, near = nullptr, far = nullptr;  // in falling priority
    cudaEvent_t swept[8] = {}, near_done[8] = {}, far_first[4] = {}, far_done[4] = {}, fork = nullptr, join = nullptr;
    std::mutex busy;
};
struct DeviceLanes {
    std::mutex build;
    bool ready = false;
    unsigned next = 0;
    PipeLane lane[4];
};

void destroy_lane(PipeLane &l) {
    for (cudaStream_t *s : {&l.tiles, &l.near, &l.far})
        if (*s) { cudaStreamDestroy(*s); *s = nullptr; }
    auto drop = [](cudaEvent_t &e) { if (e) { cudaEventDestroy(e); e = nullptr; } };
    for (auto &e : l.swept) drop(e);
    for (auto &e : l.near_done) drop(e);
    for (auto &e : l.far_first) drop(e);
    for (auto &e : l.far_done) drop(e);
    drop(l.fork);
    drop(l.join);
}

bool build_lane(PipeLane &l) {
    // the tile launches are the critical path: their CTAs go first wherever a slot frees up, then the near updates
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return false;
    const int middle = greatest + 1 <= least ? greatest + 1 : least;
    bool ok = cudaStreamCreateWithPriority(&l.tiles, cudaStreamNonBlocking, greatest) == cudaSuccess &&
              cudaStreamCreateWithPriority(&l.near, cudaStreamNonBlocking, middle) == cudaSuccess &&
              cudaStreamCreateWithPriority(&l.far, cudaStreamNonBlocking, least) == cudaSuccess &&
              cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming) == cudaSuccess;
    for (int k = 0; k < 8 && ok; ++k)
        ok = cudaEventCreateWithFlags(&l.swept[k], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&l.near_done[k], cudaEventDisableTiming) == cudaSuccess;
    for (int k = 0; k < 4 && ok; ++k)
        ok = cudaEventCreateWithFlags(&l.far_first[k], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&l.far_done[k], cudaEventDisableTiming) == cudaSuccess;
    return ok;
}

// Returns a lane of the current device with its lock held (through `held`), or null with *status set.
PipeLane *acquire_pipe_lane(cudaStream_t caller, std::unique_lock<std::mutex> &held, int *status) {
    static DeviceLanes devices[64];
    int device = 0;
    *status = G2D_ERR_CUDA;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    DeviceLanes &dl = devices[device];
    unsigned slot;
    {
        std::lock_guard<std::mutex> lock(dl.build);
        if (!dl.ready) {
            cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(caller, &capturing) != cudaSuccess) return nullptr;
            if (capturing != cudaStreamCaptureStatusNone) {
                *status = G2D_ERR_UNSUPPORTED;
                return nullptr;
            }
            bool ok = true;
            for (auto &l : dl.lane) ok = ok && build_lane(l);
            if (!ok) {
                for (auto &l : dl.lane) destroy_lane(l);
                return nullptr;
            }
            dl.ready = true;
        }
        slot = dl.next++ & 3;
    }
    held = std::unique_lock<std::mutex>(dl.lane[slot].busy);
    *status = G2D_OK;
    return &dl.lane[slot];
}

// Algorithmic flops of one near update of the pipelined schedule: the tiles of the tile anti-diagonal s as sources, the
// tiles of the anti-diagonals t0..t1 as targets, without the (source, target) pairs that the far update of the
// source's macro group carries (the same rule as band_tc_kernel's).  No padding counted.
double near_flops(int64_t m, int64_t n, int s, int t0, int t1, int outer_macro, int lag_macro) {
    const int64_t nI = ceil_div(m, TILE), nJ = ceil_div(n, TILE);
    auto extent = [](int64_t index, int64_t count, int64_t size) { return (double)(index == count - 1 ? size - index * TILE : TILE); };
    double flops = 0;
    for (int64_t TI = 0; TI < nI; ++TI)
        for (int64_t TJ = 0; TJ < nJ; ++TJ) {
            if (TI + TJ < t0 || TI + TJ > t1) continue;
            const double rows = extent(TI, nI, m), cols = extent(TJ, nJ, n);
            const int64_t w_target = (TI >> 1) + (TJ >> 1);
            const int64_t kd = s - TJ;  // down: source tile (kd, TJ)
            if (kd >= 0 && kd < TI) {
                const int64_t w_source = (kd >> 1) + (TJ >> 1);
                if (w_target < (w_source / outer_macro + 1) * outer_macro + lag_macro) flops += 2.0 * rows * cols * extent(kd, nI, m);
            }
            const int64_t kr = s - TI;  // right: source tile (TI, kr)
            if (kr >= 0 && kr < TJ) {
                const int64_t w_source = (TI >> 1) + (kr >> 1);
                if (w_target < (w_source / outer_macro + 1) * outer_macro + lag_macro) flops += 2.0 * rows * cols * extent(kr, nJ, n);
            }
        }
    return flops;
}

constexpr int kFarLagMacro = 1;  // a far update reaches the macro anti-diagonals from this many past its group's end (its first, short launch has two tile launches of time; measured against 2 and 3: less work for the near updates, the sweep 2 % shorter at 8192 x 8192 and unchanged at 2048 and 4096)

// Pipelined schedule (float, tensor cores): one tile launch per tile anti-diagonal, and the feedback between tiles
// carried by three mechanisms with growing lag, so that only the tile launches remain on the critical path:
//   * a tile hands the feedback for its lower and its right neighbour on itself: its helper warps form the two products
//     from shared memory while the tile is swept and store them into planes of their own, which the neighbours add as they
//     load one launch later;
//   * near update of the tile anti-diagonal s (its tiles as sources, targets from s + 2 on), on a side stream,
//     concurrent with the tile launch of s + 1;
//   * far update of a group of macro anti-diagonals (128 x 128 macro tiles = 2 x 2 tiles; rank 512 by default), on a
//     second side stream, into planes of its own that a tile adds when it loads.  It reaches the macro anti-diagonals
//     from kFarLagMacro past the group's end, which the tile launches get to two launches after the group's last
//     tile; the near updates stop where the far update of their source's group starts.  A far update runs as two
//     launches: first the macro anti-diagonals that the tile launches reach before the next group's update (a few
//     hundred macro tiles: short, and the only part the tile launches have to wait for soon), then everything beyond
//     them, which the tile launches only need a whole group later.
// The tile launches run on a stream of the library's own with the highest priority, the near updates below it, the far
// updates lowest: a CTA slot that frees up goes to the critical path first.  A CTA of the tile sweep fills the registers
// of two of its SM's four schedulers (six warps of up to 240 registers), so no CTA of an update kernel ever shares an SM
// with it: the updates run on the SMs that the tile launch of the moment leaves free, and the far update may as well use
// its full three-stage ring there.  Updates that share target planes are
// ordered on one stream, so the additions have a fixed order.
int sweep_pipelined(const g2d_sweep_desc *d, SweepArgs<float> &a, const TcPlanes &planes, float *yf, float *cf, cudaStream_t caller,
                    LaunchTimer *timer, double *flops) {
    std::unique_lock<std::mutex> held;
    int lane_status = G2D_OK;
    PipeLane *lane = acquire_pipe_lane(caller, held, &lane_status);
    if (!lane) return lane_status;
    // fork: everything the caller's stream holds so far comes first
    cudaStream_t stream = lane->tiles;
    if (cudaEventRecord(lane->fork, caller) != cudaSuccess || cudaStreamWaitEvent(stream, lane->fork, 0) != cudaSuccess) return G2D_ERR_CUDA;
    BandTcMaps maps;
    MacroTcMaps far_maps;
    int status = band_tc_prepare(&maps, planes, d->m, d->n);
    if (status == G2D_OK) status = macro_tc_prepare(&far_maps, planes, d->m, d->n);
    if (status != G2D_OK) return status;
    a.yf = yf; a.cf = cf; a.neighbours = 1;
    const int waves = a.nI + a.nJ - 1;
    const int waves_macro = (int)(ceil_div(d->m, MACRO) + ceil_div(d->n, MACRO)) - 1;
    const int outer = d->outer_tiles > 0 ? (d->outer_tiles + 1) / 2 : kDefaultOuterMacro;  // macro anti-diagonals per far update
    int last_near = -1, last_far = -1;
    for (int s = 0; s < waves; ++s) {
        // what the tiles of s need: every near update up to s - 2, and the far update whose first targets they are
        if (s >= 2 && last_near >= s - 2 && cudaStreamWaitEvent(stream, lane->near_done[(s - 2) & 7], 0) != cudaSuccess) return G2D_ERR_CUDA;
        if (s % 2 == 0 && s / 2 - kFarLagMacro > 0 && (s / 2 - kFarLagMacro) % outer == 0) {
            // the group that ended kFarLagMacro macro anti-diagonals ago: the first part of its update; the group before it: the rest
            const int gf = (s / 2 - kFarLagMacro) / outer - 1;
            if (last_far >= gf && cudaStreamWaitEvent(stream, lane->far_first[gf & 3], 0) != cudaSuccess) return G2D_ERR_CUDA;
            if (gf >= 1 && last_far >= gf - 1 && cudaStreamWaitEvent(stream, lane->far_done[(gf - 1) & 3], 0) != cudaSuccess) return G2D_ERR_CUDA;
        }
        if (timer) timer->begin_on(0, stream);
        status = launch_tile_sweep<float>(a, s, stream);
        if (timer) timer->end();
        if (status != G2D_OK) return status;
        const bool feeds_near = s + 2 <= waves - 1;
        // the last tiles of the macro anti-diagonal W1 - 1 lie on the tile anti-diagonal 2 W1
        const int W1 = s / 2;
        const bool feeds_far = s % 2 == 0 && W1 > 0 && W1 % outer == 0 && W1 + kFarLagMacro <= waves_macro - 1;
        if (!feeds_near && !feeds_far) continue;
        if (cudaEventRecord(lane->swept[s & 7], stream) != cudaSuccess) return G2D_ERR_CUDA;
        if (feeds_near) {
            const int reach = ((s / 2) / outer + 1) * outer + kFarLagMacro;  // of the latest group that has a source tile here
            const int t0 = s + 2, t1 = 2 * reach < waves - 1 ? 2 * reach : waves - 1;
            if (cudaStreamWaitEvent(lane->near, lane->swept[s & 7], 0) != cudaSuccess) return G2D_ERR_CUDA;
            if (timer) timer->begin_on(1, lane->near);
            status = launch_band_tc(&maps, a.y, a.c, d->m, d->n, s, s + 1, t0, t1, outer, kFarLagMacro, planes.error_flag, lane->near);
            if (timer) timer->end();
            if (status != G2D_OK) return status;
            if (flops) flops[1] += near_flops(d->m, d->n, s, t0, t1, outer, kFarLagMacro);
            if (cudaEventRecord(lane->near_done[s & 7], lane->near) != cudaSuccess) return G2D_ERR_CUDA;
            last_near = s;
        }
        if (feeds_far) {
            const int g = W1 / outer - 1;
            if (cudaStreamWaitEvent(lane->far, lane->swept[s & 7], 0) != cudaSuccess) return G2D_ERR_CUDA;
            const int t_first = W1 + kFarLagMacro, t_split = t_first + outer < waves_macro ? t_first + outer : waves_macro;
            if (timer) timer->begin_on(2, lane->far);
            status = launch_macro_update_tc(&far_maps, planes, yf, cf, d->m, d->n, W1 - outer, W1, t_split, lane->far, t_first, 3);
            if (timer) timer->end();
            if (status != G2D_OK) return status;
            if (cudaEventRecord(lane->far_first[g & 3], lane->far) != cudaSuccess) return G2D_ERR_CUDA;
            if (t_split < waves_macro) {
                if (timer) timer->begin_on(2, lane->far);
                status = launch_macro_update_tc(&far_maps, planes, yf, cf, d->m, d->n, W1 - outer, W1, waves_macro, lane->far, t_split, 3);
                if (timer) timer->end();
                if (status != G2D_OK) return status;
            }
            if (flops)
                flops[2] += band_flops(d->m, d->n, W1 - outer, W1, waves_macro, MACRO) - band_flops(d->m, d->n, W1 - outer, W1, W1 + kFarLagMacro, MACRO);
            if (cudaEventRecord(lane->far_done[g & 3], lane->far) != cudaSuccess) return G2D_ERR_CUDA;
            last_far = g;
        }
    }
    // join: what follows the call on the caller's stream follows everything the call did
    if (last_near >= 0 && cudaStreamWaitEvent(stream, lane->near_done[last_near & 7], 0) != cudaSuccess) return G2D_ERR_CUDA;
    if (last_far >= 0 && cudaStreamWaitEvent(stream, lane->far_done[last_far & 3], 0) != cudaSuccess) return G2D_ERR_CUDA;
    status = launch_sweep_finish(planes.error_flag, d->status, a.y, d->m * d->n, stream);
    if (status != G2D_OK) return status;
    if (cudaEventRecord(lane->join, stream) != cudaSuccess || cudaStreamWaitEvent(caller, lane->join, 0) != cudaSuccess) return G2D_ERR_CUDA;
    return G2D_OK;
}

template <typename F>
int sweep_fused(const g2d_sweep_desc *d, cudaStream_t stream, LaunchTimer *timer = nullptr, double *flops = nullptr) {
    const int64_t count = d->batch * d->m * d->n;
    const size_t plane = align256(sizeof(F) * (size_t)count);
    const bool tc = tc_eligible(d);
    if (!d->workspace || d->workspace_bytes < 2 * plane + (tc ? tc_extra_bytes(d) : 0)) return G2D_ERR_WORKSPACE;
    if (((uintptr_t)d->workspace & 255) != 0) return G2D_ERR_WORKSPACE;
    SweepArgs<F> a;
    a.y = (F *)d->y;
    a.c = (F *)d->workspace;
    a.e = (F *)((char *)d->workspace + plane);
    a.l = (const F *)d->l; a.u = (const F *)d->u;
    a.l_off = d->l_offsets; a.u_off = d->u_offsets;
    a.scale = (const F *)d->scale; a.zero = (const F *)d->zero;
    a.scale_off = d->scale_offsets; a.zero_off = d->zero_offsets;
    a.srs = d->scale_row_stride; a.scs = d->scale_col_stride; a.zrs = d->zero_row_stride; a.zcs = d->zero_col_stride;
    a.forced = (const F *)d->forced_z;
    a.y_pre = (F *)d->y_pre;
    a.qmin = (F)d->qmin; a.qmax = (F)d->qmax;
    a.kind = d->quant_kind;
    a.batch = d->batch; a.m = d->m; a.n = d->n;
    a.nI = (int)ceil_div(d->m, TILE); a.nJ = (int)ceil_div(d->n, TILE);
    if (cudaMemsetAsync(a.c, 0, sizeof(F) * (size_t)count, stream) != cudaSuccess) return G2D_ERR_CUDA;

    BandArgs<F> b;
    b.y = a.y; b.c = a.c; b.e = a.e; b.l = a.l; b.u = a.u; b.l_off = a.l_off; b.u_off = a.u_off;
    b.batch = a.batch; b.m = a.m; b.n = a.n; b.P = TILE; b.Q = TILE; b.down_into_y = 0; b.mode = BAND_TILE; b.filter = 0;
    if (tc) {
        // carve the operand planes behind C and E, prepare the static operands, run the macro schedule
        char *p = (char *)d->workspace + 2 * plane;
        const size_t mn = align256(4 * (size_t)d->m * d->n), mm = align256(4 * (size_t)d->m * d->m), nn = align256(4 * (size_t)d->n * d->n);
        TcPlanes planes;
        planes.error_flag = (int *)p; p += 256;
        planes.et_hi = (float *)p; p += mn; planes.et_lo = (float *)p; p += mn;
        planes.c_hi = (float *)p; p += mn; planes.c_lo = (float *)p; p += mn;
        planes.l_hi = (float *)p; p += mm; planes.l_lo = (float *)p; p += mm;
        planes.ut_hi = (float *)p; p += nn; planes.ut_lo = (float *)p; p += nn;
        if (((uintptr_t)d->y & 15) != 0) return G2D_ERR_BAD_ARGUMENT;
        if (cudaMemsetAsync(planes.error_flag, 0, sizeof(int), stream) != cudaSuccess) return G2D_ERR_CUDA;
        const int status = tc_prepare_operands((const float *)d->l, (const float *)d->u, d->m, d->n, planes, stream);
        if (status != G2D_OK) return status;
        a.et_hi = planes.et_hi; a.et_lo = planes.et_lo; a.c_hi = planes.c_hi; a.c_lo = planes.c_lo;
        if constexpr (sizeof(F) == sizeof(float)) {
            if (d->reserved == 3 || d->reserved == 0) {
                float *yf = (float *)p, *cf = (float *)(p + mn);
                a.yn = (float *)(p + 2 * mn); a.cn = (float *)(p + 3 * mn);  // written before they are read: no clearing
                if (cudaMemsetAsync(yf, 0, 2 * mn, stream) != cudaSuccess) return G2D_ERR_CUDA;
                return sweep_pipelined(d, a, planes, yf, cf, stream, timer, flops);
            }
        }
        const int swept = sweep_macro<F>(d, a, b, stream, timer, flops, &planes);
        if (swept != G2D_OK) return swept;
        return launch_sweep_finish(planes.error_flag, d->status, (float *)d->y, d->m * d->n, stream);
    }
    if (d->reserved == 2) return sweep_macro<F>(d, a, b, stream, timer, flops, nullptr);

    const int waves = a.nI + a.nJ - 1;
    const int outer = d->outer_tiles > 0 ? d->outer_tiles : kDefaultOuterTiles;
    for (int S0 = 0; S0 < waves; S0 += outer) {
        const int S1 = S0 + outer < waves ? S0 + outer : waves;
        for (int S = S0; S < S1; ++S) {
            if (timer) timer->begin(0);
            int status = launch_tile_sweep<F>(a, S, stream);
            if (timer) timer->end();
            if (status != G2D_OK) return status;
            if (S + 1 < S1) {  // near update: into the rest of the outer group
                b.s0 = S; b.s1 = S + 1; b.s_end = S1;
                if (timer) timer->begin(1);
                status = launch_band_update<F>(b, stream);
                if (timer) timer->end();
                if (flops) flops[1] += band_flops(d->m, d->n, b.s0, b.s1, b.s_end) * (double)d->batch;
                if (status != G2D_OK) return status;
            }
        }
        if (S1 < waves) {  // far update: the whole group into everything after it
            b.s0 = S0; b.s1 = S1; b.s_end = waves;
            if (timer) timer->begin(2);
            const int status = launch_band_update<F>(b, stream);
            if (timer) timer->end();
            if (flops) flops[2] += band_flops(d->m, d->n, b.s0, b.s1, b.s_end) * (double)d->batch;
            if (status != G2D_OK) return status;
        }
    }
    return G2D_OK;
}

int check_stage(const g2d_stage_desc *d) {
    if (!d) return G2D_ERR_BAD_ARGUMENT;
    if (d->dtype != G2D_F32 && d->dtype != G2D_F64) return G2D_ERR_BAD_ARGUMENT;
    if (d->batch < 0 || d->m < 0 || d->n < 0 || d->p <= 0 || d->q <= 0) return G2D_ERR_BAD_ARGUMENT;
    if (d->m % d->p || d->n % d->q) return G2D_ERR_BAD_ARGUMENT;
    return G2D_OK;
}

template <typename F>
int stage_flush(const g2d_stage_desc *d, int64_t s0, int64_t s1, int64_t s_end, cudaStream_t stream) {
    BandArgs<F> b;
    b.y = (F *)d->y; b.c = (F *)d->c; b.e = (const F *)d->e;
    b.l = (const F *)d->l; b.u = (const F *)d->u; b.l_off = d->l_offsets; b.u_off = d->u_offsets;
    b.batch = d->batch; b.m = d->m; b.n = d->n; b.P = d->p; b.Q = d->q;
    b.s0 = s0; b.s1 = s1; b.s_end = s_end; b.down_into_y = 1; b.filter = 0;
    b.mode = (d->p == 1 && d->q == 1) ? BAND_PLAIN : BAND_GENERAL;
    return launch_band_update<F>(b, stream);
}

}  // namespace

extern "C" const char *g2d_status_string(int status) {
    switch (status) {
    case G2D_OK: return "ok";
    case G2D_ERR_BAD_ARGUMENT: return "bad argument";
    case G2D_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case G2D_ERR_UNSUPPORTED: return "unsupported combination";
    case G2D_ERR_CUDA: return "CUDA runtime error";
    case G2D_ERR_TOO_LARGE: return "size exceeds a fixed maximum";
    default: return "unknown status";
    }
}

extern "C" int g2d_abi_version(void) { return 2; }

extern "C" int g2d_sweep_workspace_bytes(const g2d_sweep_desc *desc, size_t *bytes) {
    const int status = check_sweep(desc);
    if (status != G2D_OK || !bytes) return status != G2D_OK ? status : G2D_ERR_BAD_ARGUMENT;
    const size_t elem = desc->dtype == G2D_F32 ? 4 : 8;
    *bytes = 2 * align256(elem * (size_t)(desc->batch * desc->m * desc->n)) + (tc_eligible(desc) ? tc_extra_bytes(desc) : 0);
    return G2D_OK;
}

extern "C" int g2d_sweep_fused(const g2d_sweep_desc *desc, void *stream) {
    const int status = check_sweep(desc);
    if (status != G2D_OK) return status;
    if (desc->batch == 0 || desc->m == 0 || desc->n == 0) return G2D_OK;
    if (!desc->y || !desc->l || !desc->u) return G2D_ERR_BAD_ARGUMENT;
    if (desc->quant_kind == G2D_Q_AFFINE && (!desc->scale || !desc->zero || !(desc->qmin < desc->qmax))) return G2D_ERR_BAD_ARGUMENT;
    if (desc->quant_kind == G2D_Q_FORCED && !desc->forced_z) return G2D_ERR_BAD_ARGUMENT;
    if ((desc->m + TILE - 1) / TILE + (desc->n + TILE - 1) / TILE > 60000) return G2D_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    return desc->dtype == G2D_F32 ? sweep_fused<float>(desc, st) : sweep_fused<double>(desc, st);
}

extern "C" unsigned long long g2d_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int g2d_sweep_fused_profile(const g2d_sweep_desc *desc, void *stream, double *out) {
    int status = check_sweep(desc);
    if (status != G2D_OK) return status;
    if (!out) return G2D_ERR_BAD_ARGUMENT;
    for (int i = 0; i < 9; ++i) out[i] = 0;
    if (desc->batch == 0 || desc->m == 0 || desc->n == 0) return G2D_OK;
    if (!desc->y || !desc->l || !desc->u) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    LaunchTimer timer;
    timer.stream = st;
    double flops[3] = {0, 0, 0};
    status = desc->dtype == G2D_F32 ? sweep_fused<float>(desc, st, &timer, flops) : sweep_fused<double>(desc, st, &timer, flops);
    if (cudaStreamSynchronize(st) != cudaSuccess) status = status == G2D_OK ? G2D_ERR_CUDA : status;
    if (status == G2D_OK && tc_eligible(desc)) {
        // the tensor-core kernels report a bounded wait that ran out through a flag behind the C and E planes
        const size_t elem = 4, plane = align256(elem * (size_t)(desc->batch * desc->m * desc->n));
        int flag = 0;
        if (cudaMemcpy(&flag, (const char *)desc->workspace + 2 * plane, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess || flag != 0)
            status = G2D_ERR_CUDA;
    }
    for (auto &it : timer.items) {
        float ms = 0;
        if (status == G2D_OK && timer.ok && cudaEventElapsedTime(&ms, it.begin, it.end) == cudaSuccess) {
            out[it.kind] += ms;
            out[3 + it.kind] += 1;
        }
        if (it.begin) cudaEventDestroy(it.begin);
        if (it.end) cudaEventDestroy(it.end);
    }
    out[7] = flops[1];
    out[8] = flops[2];
    const double mm = (double)desc->m, nn = (double)desc->n;
    out[6] = mm * nn * (mm + nn - 2) * (double)desc->batch;  // algorithmic flops of the whole sweep
    if (!timer.ok && status == G2D_OK) status = G2D_ERR_CUDA;
    return status;
}

extern "C" int g2d_stage_push(const g2d_stage_desc *desc, const void *z, int64_t s, int64_t s1, void *stream) {
    const int status = check_stage(desc);
    if (status != G2D_OK) return status;
    if (desc->batch == 0 || desc->m == 0 || desc->n == 0) return G2D_OK;
    if (!desc->y || !desc->c || !desc->e || !desc->l || !desc->u || !z) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    return desc->dtype == G2D_F32 ? launch_stage_push<float>(*desc, (const float *)z, s, s1, st)
                                  : launch_stage_push<double>(*desc, (const double *)z, s, s1, st);
}

extern "C" int g2d_stage_flush(const g2d_stage_desc *desc, int64_t s0, int64_t s1, int64_t s_end, void *stream) {
    const int status = check_stage(desc);
    if (status != G2D_OK) return status;
    if (desc->batch == 0 || desc->m == 0 || desc->n == 0) return G2D_OK;
    if (!desc->y || !desc->c || !desc->e || !desc->l || !desc->u) return G2D_ERR_BAD_ARGUMENT;
    if (s0 < 0 || s1 <= s0 || s_end < s1) return G2D_ERR_BAD_ARGUMENT;
    if (s_end == s1) return G2D_OK;
    cudaStream_t st = (cudaStream_t)stream;
    return desc->dtype == G2D_F32 ? stage_flush<float>(desc, s0, s1, s_end, st) : stage_flush<double>(desc, s0, s1, s_end, st);
}
