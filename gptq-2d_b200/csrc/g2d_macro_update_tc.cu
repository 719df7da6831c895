// Feedback between macro tiles on the tensor cores (float only): tcgen05.mma kind::tf32 with accumulators in
// tensor memory, operands brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle).
//
// One CTA owns one 128 x 128 target macro tile and forms both products of the band update
//     down :  C[I, J] += sum_k L[I, k] E[k, J]      right:  Y[I, J] += sum_k C[I, k] U[k, J]
// over the k ranges that hold the sources of the macro anti-diagonals s0..s1-1 (whole 128-blocks, no masks).
// fp32 fidelity comes from the 3xTF32 split: every operand exists as hi = tf32(a) and lo = a - hi, and each
// k step issues hi*hi + lo*hi + hi*lo into the same fp32 accumulator.  All four operand kinds are stored K-major
// for the MMA: L and C as they are (rows x k), E and U transposed (columns x k); the split copies of L and U^T are
// made once per sweep by the kernels at the end of this file, those of E^T and C by the tile sweep as it finishes
// a tile.
//
// Warp roles (6 warps): warp 0 issues the TMA loads, warp 1 allocates tensor memory and issues the MMAs,
// warps 2-5 read the accumulators (each its own 32 lanes) and add them into C / Y.  A three-stage ring of
// 64 KB (A_hi, A_lo, B_hi, B_lo tiles of 128 x 32) is handed over with mbarriers; tcgen05.commit releases a stage
// when its MMAs have read it.  Every wait is bounded: on time-out a flag is set and the CTA winds down.
#include "g2d_tc.cuh"

namespace g2d {

constexpr int RB_I = 8, RB_J = 16;  // rasterisation block of the far updates: 128 macro tiles, about one wave of CTAs

struct TcMaps {
    CUtensorMap l_hi, l_lo, c_hi, c_lo;      // A operands: [rows][k]
    CUtensorMap et_hi, et_lo, ut_hi, ut_lo;  // B operands: [columns][k]
};

template <int NSTAGES>
__global__ void __launch_bounds__(TC_THREADS) macro_update_tc_kernel(const __grid_constant__ TcMaps maps, float *y, float *c, int64_t m,
                                                                     int64_t n, int nI2, int nJ2, int s0, int s1, int t_first, int s_end,
                                                                     int raster, int *error_flag) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[NSTAGES], empty_bar[NSTAGES], accum_bar[2];  // one accumulator barrier per product
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    // Target macro tile.  With gridDim.y > 1, blockIdx.y selects the macro anti-diagonal and blockIdx.x the tile on it
    // (few anti-diagonals: near updates).  Otherwise the whole macro grid is walked in RB_I x RB_J blocks, so that the
    // CTAs resident at one time cover a compact patch and share their L / C row strips and E^T / U^T column strips in L2.
    int I2, J2;
    if (raster == 0) {
        const int W = t_first + (int)blockIdx.y;
        const int ti_lo = max(0, W - nJ2 + 1), ti_hi = min(W + 1, nI2);
        I2 = ti_lo + (int)blockIdx.x;
        if (W >= s_end || I2 >= ti_hi) return;
        J2 = W - I2;
    } else {
        const int blocks_j = (nJ2 + RB_J - 1) / RB_J;
        const int blk = (int)blockIdx.x / (RB_I * RB_J), within = (int)blockIdx.x % (RB_I * RB_J);
        I2 = (blk / blocks_j) * RB_I + within / RB_J;
        J2 = (blk % blocks_j) * RB_J + within % RB_J;
        if (I2 >= nI2 || J2 >= nJ2 || I2 + J2 < t_first || I2 + J2 >= s_end) return;
    }
    // source macro rows (down) and macro columns (right) of the band
    const int kd_lo = max(s0 - J2, 0), kd_hi = min(s1 - J2, I2);
    const int kr_lo = max(s0 - I2, 0), kr_hi = min(s1 - I2, J2);
    const int chunks_d = kd_hi > kd_lo ? (kd_hi - kd_lo) * (MT / KC) : 0;
    const int chunks_r = kr_hi > kr_lo ? (kr_hi - kr_lo) * (MT / KC) : 0;
    const int chunks = chunks_d + chunks_r;
    if (chunks == 0) return;

    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar[0], 1);
        mbar_init(&accum_bar[1], 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    const int i0 = I2 * MT, j0 = J2 * MT;

    if (warp == 0) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % NSTAGES, round = ch / NSTAGES;
                if (round > 0 && !mbar_wait(&empty_bar[stage], (round - 1) & 1)) { failed = 1; break; }
                const bool down = ch < chunks_d;
                const int k = down ? kd_lo * MT + ch * KC : kr_lo * MT + (ch - chunks_d) * KC;
                const uint32_t dst = smem_base + stage * STAGE_BYTES;
                mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
                tma_load_2d(dst, down ? &maps.l_hi : &maps.c_hi, k, i0, &full_bar[stage]);
                tma_load_2d(dst + TILE_BYTES, down ? &maps.l_lo : &maps.c_lo, k, i0, &full_bar[stage]);
                tma_load_2d(dst + 2 * TILE_BYTES, down ? &maps.et_hi : &maps.ut_hi, k, j0, &full_bar[stage]);
                tma_load_2d(dst + 3 * TILE_BYTES, down ? &maps.et_lo : &maps.ut_lo, k, j0, &full_bar[stage]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int ch = 0; ch < chunks && ok; ++ch) {
                const int stage = ch % NSTAGES, round = ch / NSTAGES;
                if (!mbar_wait(&full_bar[stage], round & 1)) { failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const bool down = ch < chunks_d;
                const uint32_t d_addr = tmem + (down ? 0u : (uint32_t)MT);
                const bool first = down ? ch == 0 : ch == chunks_d;
                const uint32_t a_hi = smem_base + stage * STAGE_BYTES, a_lo = a_hi + TILE_BYTES, b_hi = a_hi + 2 * TILE_BYTES,
                               b_lo = a_hi + 3 * TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < KC / 8; ++ks) {
                    const uint32_t off = ks * 32;  // 8 tf32 values = 32 bytes along the swizzled row
                    umma_tf32(d_addr, umma_desc(a_hi + off), umma_desc(b_hi + off), IDESC, (first && ks == 0) ? 0u : 1u);
                    umma_tf32(d_addr, umma_desc(a_lo + off), umma_desc(b_hi + off), IDESC, 1u);
                    umma_tf32(d_addr, umma_desc(a_hi + off), umma_desc(b_lo + off), IDESC, 1u);
                }
                umma_commit(&empty_bar[stage]);  // arrives when the MMAs above have read the stage
                // the down product is complete with its last chunk: its accumulator is read out and added to C by the
                // epilogue warps while the MMAs of the right product run into the other accumulator
                if (ch == chunks_d - 1) umma_commit(&accum_bar[0]);
            }
            if (ok && chunks_r > 0) umma_commit(&accum_bar[1]);  // arrives when every MMA issued so far has completed
        }
    } else {
        // epilogue warps: lanes 32 q .. 32 q + 31 of tensor memory, q = warp % 4
        const int q = warp & 3;
        const int64_t row = (int64_t)i0 + q * 32 + lane;
        bool go = true;
        {
            for (int prod = 0; prod < 2 && go; ++prod) {
                if ((prod == 0 ? chunks_d : chunks_r) == 0) continue;
                const bool ok = mbar_wait(&accum_bar[prod], 0, 256);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!ok) failed = 1;
                go = __all_sync(0xffffffffu, ok && !failed);  // warp-uniform: the tensor-memory loads are warp-wide
                if (!go) break;
                float *plane = prod == 0 ? c : y;
                for (int cb = 0; cb < MT / 32; ++cb) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(prod * MT + cb * 32);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row < m) {
                        float *p = plane + row * n + j0 + cb * 32;
#pragma unroll
                        for (int x = 0; x < 32; x += 4) {
                            if ((int64_t)j0 + cb * 32 + x < n) {  // n is a multiple of 4: a group is inside or outside as a whole
                                // one CTA owns each target entry, so the reduction needs no read-back and stays deterministic
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + x), "f"(__uint_as_float(v[x])),
                                             "f"(__uint_as_float(v[x + 1])), "f"(__uint_as_float(v[x + 2])), "f"(__uint_as_float(v[x + 3]))
                                             : "memory");
                            }
                        }
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
            if (lane == 0) mbar_wait(&accum_bar[chunks_r > 0 ? 1 : 0], 0);
            __syncwarp();
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && error_flag) atomicExch(error_flag, 1);
}

// ---- one-time operand preparation ---------------------------------------------------------------------

// L (row-major, read strictly below the diagonal) -> hi / lo copies with zeros elsewhere
__global__ void split_lower_kernel(const float *__restrict__ l, int64_t m, float *__restrict__ hi, float *__restrict__ lo) {
    const int64_t total = m * m;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / m, cidx = t % m;
        float h = 0.f, o = 0.f;
        if (cidx < r) split_tf32(l[t], h, o);
        hi[t] = h;
        lo[t] = o;
    }
}

// U (row-major, read strictly above the diagonal) -> transposed hi / lo copies: out[j][k] = U[k][j] for k < j
__global__ void split_upper_transposed_kernel(const float *__restrict__ u, int64_t n, float *__restrict__ hi, float *__restrict__ lo) {
    __shared__ float tile[32][33];
    const int64_t tiles = ceil_div(n, 32);
    for (int64_t b = blockIdx.x; b < tiles * tiles; b += gridDim.x) {
        const int64_t k0 = (b / tiles) * 32, j0 = (b % tiles) * 32;  // source block: rows k, columns j
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t k = k0 + r, j = j0 + threadIdx.x;
            tile[r][threadIdx.x] = (k < n && j < n && k < j) ? u[k * n + j] : 0.f;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t j = j0 + r, k = k0 + threadIdx.x;
            if (j < n && k < n) {
                float h, o;
                split_tf32(tile[threadIdx.x][r], h, o);
                hi[j * n + k] = h;
                lo[j * n + k] = o;
            }
        }
        __syncthreads();
    }
}

// ---- host side ---------------------------------------------------------------------------------------

int tc_prepare_operands(const float *l, const float *u, int64_t m, int64_t n, const TcPlanes &pl, cudaStream_t stream) {
    split_lower_kernel<<<148 * 8, 256, 0, stream>>>(l, m, pl.l_hi, pl.l_lo);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    split_upper_transposed_kernel<<<148 * 8, dim3(32, 8), 0, stream>>>(u, n, pl.ut_hi, pl.ut_lo);
    return check_launch();
}

// Sources: the macro anti-diagonals s0..s1-1; targets: t_first..s_end-1 (t_first >= s1).  `stages` 3 is the full pipeline
// (one CTA per SM); 2 leaves shared memory for CTAs of other kernels beside it.
static_assert(sizeof(TcMaps) <= sizeof(MacroTcMaps), "opaque tensor-map storage is too small");

// Tensor maps of one sweep (encoded once, reused by every macro update of the sweep) and the kernels' one-time set-up.
int macro_tc_prepare(MacroTcMaps *opaque, const TcPlanes &pl, int64_t m, int64_t n) {
    TcMaps &maps = *reinterpret_cast<TcMaps *>(opaque);
    if (!make_map(&maps.l_hi, pl.l_hi, m, m) || !make_map(&maps.l_lo, pl.l_lo, m, m) || !make_map(&maps.c_hi, pl.c_hi, m, n) ||
        !make_map(&maps.c_lo, pl.c_lo, m, n) || !make_map(&maps.et_hi, pl.et_hi, n, m) || !make_map(&maps.et_lo, pl.et_lo, n, m) ||
        !make_map(&maps.ut_hi, pl.ut_hi, n, n) || !make_map(&maps.ut_lo, pl.ut_lo, n, n))
        return G2D_ERR_CUDA;
    static PerDeviceOnce configured;
    return configured.run([&] {
        return cudaFuncSetAttribute(macro_update_tc_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * STAGE_BYTES + 1024) == cudaSuccess &&
               cudaFuncSetAttribute(macro_update_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * STAGE_BYTES + 1024) == cudaSuccess;
    });
}

int launch_macro_update_tc(const MacroTcMaps *opaque, const TcPlanes &pl, float *y, float *c, int64_t m, int64_t n, int s0, int s1, int s_end,
                           cudaStream_t stream, int t_first, int stages) {
    const TcMaps &maps = *reinterpret_cast<const TcMaps *>(opaque);
    if (t_first < s1) t_first = s1;
    const int depth = stages == 2 ? 2 : STAGES;
    const size_t smem = (size_t)depth * STAGE_BYTES + 1024;
    const int nI2 = (int)ceil_div(m, MT), nJ2 = (int)ceil_div(n, MT);
    if (s_end <= t_first) return G2D_OK;
    const int raster = s_end - t_first > 8 ? 1 : 0;
    dim3 grid((unsigned)(nI2 < nJ2 ? nI2 : nJ2), (unsigned)(s_end - t_first));
    if (raster) {
        const int64_t blocks = ceil_div(nI2, RB_I) * ceil_div(nJ2, RB_J);
        grid = dim3((unsigned)(blocks * RB_I * RB_J), 1);
    }
    if (depth == 2)
        macro_update_tc_kernel<2><<<grid, TC_THREADS, smem, stream>>>(maps, y, c, m, n, nI2, nJ2, s0, s1, t_first, s_end, raster, pl.error_flag);
    else
        macro_update_tc_kernel<STAGES><<<grid, TC_THREADS, smem, stream>>>(maps, y, c, m, n, nI2, nJ2, s0, s1, t_first, s_end, raster, pl.error_flag);
    return check_launch();
}

}  // namespace g2d
