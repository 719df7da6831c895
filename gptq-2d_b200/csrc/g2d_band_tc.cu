// Feedback between tiles on the tensor cores for the pipelined schedule (float only).
//
// A band update carries the finished tiles of the tile anti-diagonals s0..s1-1 (sources) into the tiles of the
// anti-diagonals t0..t1 (targets), t0 >= s1 + 1:
//     down :  C[I, J] += sum_k L[I, k] E[k, J],   k = s - J for the sources s      (same column of tiles)
//     right:  Y[I, J] += sum_k C[I, k] U[k, J],   k = s - I for the sources s      (same row of tiles)
// The k range of a target depends on its column (down) or its row (right) only, so a CTA takes two tiles that share
// it: a down job owns 128 rows x 64 columns (tile rows I, I + 1 of column J), a right job 64 rows x 128 columns, the
// latter formed transposed (Y^T = U^T C^T) so that the 128 side is again the M side of the MMA.  Each product is a
// tcgen05.mma kind::tf32 with M = 128, N = 64 and the 3xTF32 split; operands are the K-major hi / lo planes that the
// macro updates use (L and U^T split once per sweep, E^T and C by the tile sweep as it finishes a tile).
// Every target entry is owned by one CTA of one launch, launches that share targets are ordered by the caller, and
// the additions are reductions in global memory: the result does not depend on scheduling.
#include "g2d_tc.cuh"

namespace g2d {

constexpr int BN = 64;                               // N of the MMA: one tile
constexpr int B_TILE_BYTES = BN * KC * 4;            // 8 KB
constexpr int BAND_STAGE_BYTES = 2 * TILE_BYTES + 2 * B_TILE_BYTES;  // A_hi, A_lo, B_hi, B_lo
constexpr int BAND_STAGES = 1;  // 48 KB: the updates are short and latency-bound, so several CTAs per SM
constexpr uint32_t BAND_TMEM_COLS = 64;
// D fp32, A and B tf32, both K-major, M = 128, N = 64
constexpr uint32_t IDESC_N64 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(MT >> 4) << 24);

struct BandJob {
    CUtensorMap l_hi, l_lo, ut_hi, ut_lo;  // A operands: boxes of 128 rows
    CUtensorMap et_hi, et_lo, c_hi, c_lo;  // B operands: boxes of 64 rows
    float *y, *c;                          // planes that receive the right and the down feedback
    int64_t m, n;
    int nI, nJ;                            // tiles per column / per row
    int s0, s1, t0, t1;
    int outer_macro, lag_macro;            // > 0: targets that the far update of the source's macro group reaches are left out
    int *error_flag;
};

// grid: x = tile column (down jobs) or tile row (right jobs), y = pair slot along the target range, z = 0 down, 1 right
__global__ void __launch_bounds__(TC_THREADS) band_tc_kernel(const __grid_constant__ BandJob job) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[BAND_STAGES], empty_bar[BAND_STAGES], accum_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    const bool right = blockIdx.z != 0;
    const int fixed = blockIdx.x;                        // J (down) or I (right)
    const int fixed_count = right ? job.nI : job.nJ, moving_count = right ? job.nJ : job.nI;
    if (fixed >= fixed_count) return;
    const int first = max(job.t0 - fixed, 0);
    const int pair = (first >> 1) + (int)blockIdx.y;     // tiles 2 pair, 2 pair + 1 along the moving index
    const int t_a = 2 * pair, t_b = 2 * pair + 1;
    bool valid_a = t_a < moving_count && t_a + fixed >= job.t0 && t_a + fixed <= job.t1;
    bool valid_b = t_b < moving_count && t_b + fixed >= job.t0 && t_b + fixed <= job.t1;
    if (!valid_a && !valid_b) return;
    // source tiles along k: diagonals s0..s1-1 in this column / row; all of them lie before both targets
    const int k_lo = max(job.s0 - fixed, 0), k_hi = min(job.s1 - fixed, moving_count);
    if (k_hi <= k_lo) return;
    if (job.outer_macro > 0) {
        // one source diagonal: one source tile (k_lo, fixed); both targets lie in one macro tile
        const int w_source = (k_lo >> 1) + (fixed >> 1), w_target = pair + (fixed >> 1);
        const int reach = (w_source / job.outer_macro + 1) * job.outer_macro + job.lag_macro;  // the far update starts here
        if (w_target >= reach) return;
    }
    const int chunks = (k_hi - k_lo) * (TILE / KC);
    const int a_row = t_a * TILE;                        // first of the 128 rows of the A operand
    const int b_row = fixed * TILE;                      // first of the 64 rows of the B operand
    const CUtensorMap *a_hi = right ? &job.ut_hi : &job.l_hi, *a_lo = right ? &job.ut_lo : &job.l_lo;
    const CUtensorMap *b_hi = right ? &job.c_hi : &job.et_hi, *b_lo = right ? &job.c_lo : &job.et_lo;

    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < BAND_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(BAND_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % BAND_STAGES, round = ch / BAND_STAGES;
                if (round > 0 && !mbar_wait(&empty_bar[stage], (round - 1) & 1)) { failed = 1; break; }
                const int k = k_lo * TILE + ch * KC;
                const uint32_t dst = smem_base + stage * BAND_STAGE_BYTES;
                mbar_expect_tx(&full_bar[stage], BAND_STAGE_BYTES);
                tma_load_2d(dst, a_hi, k, a_row, &full_bar[stage]);
                tma_load_2d(dst + TILE_BYTES, a_lo, k, a_row, &full_bar[stage]);
                tma_load_2d(dst + 2 * TILE_BYTES, b_hi, k, b_row, &full_bar[stage]);
                tma_load_2d(dst + 2 * TILE_BYTES + B_TILE_BYTES, b_lo, k, b_row, &full_bar[stage]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % BAND_STAGES, round = ch / BAND_STAGES;
                if (!mbar_wait(&full_bar[stage], round & 1)) { failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t s_a_hi = smem_base + stage * BAND_STAGE_BYTES, s_a_lo = s_a_hi + TILE_BYTES, s_b_hi = s_a_hi + 2 * TILE_BYTES,
                               s_b_lo = s_b_hi + B_TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < KC / 8; ++ks) {
                    const uint32_t off = ks * 32;  // 8 tf32 values = 32 bytes along the swizzled row
                    umma_tf32(tmem, umma_desc(s_a_hi + off), umma_desc(s_b_hi + off), IDESC_N64, (ch == 0 && ks == 0) ? 0u : 1u);
                    umma_tf32(tmem, umma_desc(s_a_lo + off), umma_desc(s_b_hi + off), IDESC_N64, 1u);
                    umma_tf32(tmem, umma_desc(s_a_hi + off), umma_desc(s_b_lo + off), IDESC_N64, 1u);
                }
                umma_commit(&empty_bar[stage]);  // arrives when the MMAs above have read the stage
            }
            umma_commit(&accum_bar);             // arrives when every MMA issued so far has completed
        }
    } else {
        // epilogue warps: lanes 32 q .. 32 q + 31 of tensor memory, q = warp % 4; lanes 0-63 belong to tile a, 64-127 to tile b
        const int q = warp & 3;
        const bool ok = mbar_wait(&accum_bar, 0, 256);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!ok) failed = 1;
        const bool go = __all_sync(0xffffffffu, ok && !failed);  // warp-uniform: the tensor-memory loads are warp-wide
        const bool mine = q < 2 ? valid_a : valid_b;             // warp-uniform as well
        if (go && mine) {
            const int64_t along = (int64_t)a_row + q * 32 + lane;  // row (down) or column (right) of this lane
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t v[32];
                tmem_load_32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), v);
                const int64_t across0 = (int64_t)b_row + cb * 32;  // first column (down) or row (right) of the 32 values
                if (!right) {
                    if (along < job.m) {
                        float *p = job.c + along * job.n + across0;
#pragma unroll
                        for (int x = 0; x < 32; x += 4) {
                            if (across0 + x < job.n) {  // n is a multiple of 4: a group is inside or outside as a whole
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + x), "f"(__uint_as_float(v[x])),
                                             "f"(__uint_as_float(v[x + 1])), "f"(__uint_as_float(v[x + 2])), "f"(__uint_as_float(v[x + 3]))
                                             : "memory");
                            }
                        }
                    }
                } else if (along < job.n) {
                    // transposed product: consecutive lanes hold consecutive columns of one row of Y
                    float *p = job.y + across0 * job.n + along;
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        if (across0 + x < job.m)
                            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p + (int64_t)x * job.n), "f"(__uint_as_float(v[x])) : "memory");
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        if (failed) {
            // give outstanding loads and MMAs a bounded chance to land before the memory they target is released
            if (lane == 0) mbar_wait(&accum_bar, 0);
            __syncwarp();
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BAND_TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && job.error_flag) atomicExch(job.error_flag, 1);
}

// Tensor maps of one sweep; encoded once and reused by every band launch.
struct BandMaps {
    CUtensorMap l_hi, l_lo, ut_hi, ut_lo, et_hi, et_lo, c_hi, c_lo;
};
static_assert(sizeof(BandMaps) <= sizeof(BandTcMaps), "opaque tensor-map storage is too small");

int band_tc_prepare(BandTcMaps *opaque, const TcPlanes &pl, int64_t m, int64_t n) {
    BandMaps *maps = reinterpret_cast<BandMaps *>(opaque);
    if (!make_map(&maps->l_hi, pl.l_hi, m, m) || !make_map(&maps->l_lo, pl.l_lo, m, m) || !make_map(&maps->ut_hi, pl.ut_hi, n, n) ||
        !make_map(&maps->ut_lo, pl.ut_lo, n, n) || !make_map(&maps->et_hi, pl.et_hi, n, m, BN) || !make_map(&maps->et_lo, pl.et_lo, n, m, BN) ||
        !make_map(&maps->c_hi, pl.c_hi, m, n, BN) || !make_map(&maps->c_lo, pl.c_lo, m, n, BN))
        return G2D_ERR_CUDA;
    static PerDeviceOnce configured;
    // Several CTAs of this kernel share an SM, with one another and with other kernels' CTAs.  It asks for the largest
    // shared-memory carve-out: an SM that a kernel with a smaller one had configured takes no CTA beside it that needs
    // more until it has drained.
    return configured.run([&] {
        return cudaFuncSetAttribute(band_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BAND_STAGES * BAND_STAGE_BYTES + 1024) == cudaSuccess &&
               cudaFuncSetAttribute(band_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) == cudaSuccess;
    });
}

int launch_band_tc(const BandTcMaps *opaque, float *y, float *c, int64_t m, int64_t n, int s0, int s1, int t0, int t1, int outer_macro,
                   int lag_macro, int *error_flag, cudaStream_t stream) {
    const BandMaps *maps = reinterpret_cast<const BandMaps *>(opaque);
    BandJob job;
    job.l_hi = maps->l_hi; job.l_lo = maps->l_lo; job.ut_hi = maps->ut_hi; job.ut_lo = maps->ut_lo;
    job.et_hi = maps->et_hi; job.et_lo = maps->et_lo; job.c_hi = maps->c_hi; job.c_lo = maps->c_lo;
    job.y = y; job.c = c; job.m = m; job.n = n;
    job.nI = (int)ceil_div(m, (int64_t)TILE); job.nJ = (int)ceil_div(n, (int64_t)TILE);
    const int waves = job.nI + job.nJ - 1;
    if (t1 > waves - 1) t1 = waves - 1;
    if (t0 < s1 + 1 || t1 < t0 || s1 <= s0) return t1 < t0 || s1 <= s0 ? G2D_OK : G2D_ERR_BAD_ARGUMENT;
    job.s0 = s0; job.s1 = s1; job.t0 = t0; job.t1 = t1;
    job.outer_macro = s1 == s0 + 1 ? outer_macro : 0; job.lag_macro = lag_macro;
    job.error_flag = error_flag;
    // pairs along the moving index that can hold a target: at most (t1 - t0) / 2 + 2, never more than the matrix has
    const int longest = job.nI > job.nJ ? job.nI : job.nJ;
    int slots = (t1 - t0) / 2 + 2;
    if (slots > (longest + 1) / 2) slots = (longest + 1) / 2;
    dim3 grid((unsigned)longest, (unsigned)slots, 2);
    band_tc_kernel<<<grid, TC_THREADS, BAND_STAGES * BAND_STAGE_BYTES + 1024, stream>>>(job);
    return check_launch();
}

}  // namespace g2d
