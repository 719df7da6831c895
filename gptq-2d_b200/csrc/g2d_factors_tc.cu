// The two bulk products of the factor preparation on the tensor cores (float only): the trailing update of the
// blocked Cholesky factorization (second half of this file) and the triangular inverse.
//
// The inverse Lf = T^{-1} of the lower triangular Cholesky factor is built by doubling: at level b every aligned pair
// of finished b x b diagonal blocks [A^{-1} 0; . B^{-1}] of Lf is completed by X = -B^{-1} (C A^{-1}) with
// C = T[second half rows, first half columns].  From b = 128 on, both products of a level run here as tcgen05.mma
// kind::tf32 GEMMs over 128 x 128 output tiles on three tf32 planes per operand (six products per k step, see
// "Precision" below).  The MMA wants both operands K-major, so the first product is formed transposed,
//     W^T[j][i] = sum_k Lf^T[j][k] T[i][k]        (k from the tile's first row j0 to the end of the first half)
//     X[i][j]   = -sum_k Lf[i][k] W^T[j][k]       (k from the start of the second half through the tile's rows)
// and every operand is kept as ready-made hi / mid / lo planes: Lf and its transpose (both written by the second
// product's epilogue), and one plane triple whose lower triangle holds T and whose upper triangle receives W^T.
// Same pipeline as the macro updates of the sweep: one warp issues TMA loads into a two-stage ring of 96 KB stages, one
// warp issues the MMAs, four warps read the accumulators and store; every wait is bounded.
#include <cstring>

#include "g2d_tc.cuh"

namespace g2d {

struct FactorMaps {
    CUtensorMap out[3], outt[3], tw[3];  // hi, mid, lo
};
struct TrinvJob {
    FactorMaps maps[2];
    FactorPlanes p[2];
    int pairs;   // pairs of diagonal blocks of the largest problem; blockIdx.x = problem * pairs + pair
    int tiles;   // b / 128
    int64_t b;
    int second;  // 0: W^T, 1: X
};

// Precision.  The inverse is where a badly conditioned factor shows: every level multiplies explicit inverse blocks, and
// the error of each product is amplified by the cancellation in -B^{-1} (C A^{-1}); with the two-plane 3xTF32 split
// (2^-21 per product) the factors of a heavy-tailed, 1 %-damped 4096 x 4096 Gram came out 4e-5 from the float64 result
// where a float32 LAPACK factorization is 1.5e-6 away.  So this kernel uses three planes per operand and six products
// (about 2^-32 per product), and keeps the one large product (hi hi') in an accumulator of its own, so that the five
// small ones are not truncated against it.  What then remained (1.4e-5 at 4096, growing with n where the same algorithm
// on FFMA stays at 2.4e-6) was the tensor cores' accumulation itself: every add into the float accumulator truncates, and
// the sums here run over up to n / 2 terms.  So the k range is cut into slices of 256: each slice is accumulated in
// tensor memory, and the epilogue warps add the slices up in registers with round-to-nearest additions while the MMAs
// of the next slice run into a second pair of accumulators.
constexpr int TRINV_STAGES = 2;
constexpr int TRINV_STAGE_BYTES = 6 * TILE_BYTES;          // A hi, mid, lo; B hi, mid, lo
constexpr int TRINV_SLICE = 8;                             // chunks per slice: k = 256
constexpr uint32_t TRINV_TMEM_COLS = 4 * MT;               // two alternating pairs of (main, correction) accumulators

__device__ __forceinline__ void trinv_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(TC_THREADS) trinv_tc_kernel(const __grid_constant__ TrinvJob job) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) TcRing ring;
    __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
    const int z = (int)blockIdx.x >= job.pairs ? 1 : 0;
    const int64_t pair = (int64_t)blockIdx.x - (int64_t)z * job.pairs;
    const FactorPlanes P = z ? job.p[1] : job.p[0];
    const FactorMaps *maps = z ? &job.maps[1] : &job.maps[0];
    const int64_t n = P.n, b = job.b;
    const int64_t r0 = pair * 2 * b, r1 = r0 + b;  // first half rows [r0, r1), second half rows [r1, r2)
    if (r1 >= n) return;
    const int64_t r2 = min(r0 + 2 * b, n);
    // output tile: rows m0.. of the A operand's matrix, columns n0.. of the B operand's
    int64_t m0, n0, k_lo, k_hi;
    const CUtensorMap *a_maps;
    if (!job.second) {
        m0 = r0 + (int64_t)blockIdx.z * MT;  // j: long k ranges (small j) are scheduled first
        n0 = r1 + (int64_t)blockIdx.y * MT;  // i
        if (n0 >= r2) return;
        k_lo = m0;
        k_hi = r1;
        a_maps = maps->outt;
    } else {
        m0 = r1 + (int64_t)(job.tiles - 1 - (int)blockIdx.y) * MT;  // i: long k ranges (large i) first
        if (m0 >= r2) return;
        n0 = r0 + (int64_t)blockIdx.z * MT;  // j
        k_lo = r1;
        k_hi = min(m0 + MT, r2);
        a_maps = maps->out;
    }
    const int chunks = (int)ceil_div(k_hi - k_lo, (int64_t)KC);  // a ragged tail reads zeros beyond the matrix
    const int slices = (chunks + TRINV_SLICE - 1) / TRINV_SLICE;

    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s2 = 0; s2 < 2; ++s2) {
            mbar_init(&acc_full[s2], 1);
            mbar_init(&acc_empty[s2], 4);  // one arrival per epilogue warp
        }
    }
    const uint32_t tmem = tc_ring_setup(ring, TRINV_TMEM_COLS);  // fences the barrier initialisations and synchronises the CTA
    if (warp == 0) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % TRINV_STAGES, round = ch / TRINV_STAGES;
                if (round > 0 && !mbar_wait(&ring.empty[stage], (round - 1) & 1)) {
                    ring.failed = 1;
                    break;
                }
                const int k = (int)(k_lo + (int64_t)ch * KC);
                const uint32_t dst = smem_base + stage * TRINV_STAGE_BYTES;
                mbar_expect_tx(&ring.full[stage], TRINV_STAGE_BYTES);
                for (int part = 0; part < 3; ++part) {
                    tma_load_2d(dst + part * TILE_BYTES, &a_maps[part], k, (int)m0, &ring.full[stage]);
                    tma_load_2d(dst + (3 + part) * TILE_BYTES, &maps->tw[part], k, (int)n0, &ring.full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % TRINV_STAGES, round = ch / TRINV_STAGES;
                const int slice = ch / TRINV_SLICE, buf = slice & 1;
                const bool opens = ch % TRINV_SLICE == 0, closes = ch % TRINV_SLICE == TRINV_SLICE - 1 || ch == chunks - 1;
                // the accumulators must have been read out by the epilogue of the slice two before
                if (opens && slice >= 2 && !mbar_wait(&acc_empty[buf], ((slice >> 1) - 1) & 1)) {
                    ring.failed = 1;
                    break;
                }
                if (!mbar_wait(&ring.full[stage], round & 1)) {
                    ring.failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc_main = tmem + (uint32_t)(buf * 2 * MT), acc_small = acc_main + MT;
                const uint32_t base = smem_base + stage * TRINV_STAGE_BYTES;
                const uint32_t a_hi = base, a_mid = base + TILE_BYTES, a_lo = base + 2 * TILE_BYTES;
                const uint32_t b_hi = base + 3 * TILE_BYTES, b_mid = base + 4 * TILE_BYTES, b_lo = base + 5 * TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < KC / 8; ++ks) {
                    const uint32_t off = ks * 32;  // 8 tf32 values = 32 bytes along the swizzled row
                    const uint32_t fresh = (opens && ks == 0) ? 0u : 1u;
                    umma_tf32(acc_main, umma_desc(a_hi + off), umma_desc(b_hi + off), IDESC, fresh);
                    umma_tf32(acc_small, umma_desc(a_hi + off), umma_desc(b_mid + off), IDESC, fresh);
                    umma_tf32(acc_small, umma_desc(a_mid + off), umma_desc(b_hi + off), IDESC, 1u);
                    umma_tf32(acc_small, umma_desc(a_mid + off), umma_desc(b_mid + off), IDESC, 1u);
                    umma_tf32(acc_small, umma_desc(a_hi + off), umma_desc(b_lo + off), IDESC, 1u);
                    umma_tf32(acc_small, umma_desc(a_lo + off), umma_desc(b_hi + off), IDESC, 1u);
                }
                umma_commit(&ring.empty[stage]);            // arrives when the MMAs above have read the stage
                if (closes) umma_commit(&acc_full[buf]);    // arrives when the slice is complete in tensor memory
            }
            umma_commit(&ring.accum);                       // arrives when every MMA issued so far has completed
        }
    } else {
        // epilogue warps: lanes 32 q .. 32 q + 31 of tensor memory, q = warp % 4; one accumulator row per thread, whose
        // 128 running sums stay in registers across the slices
        const int q = warp & 3;
        float total[MT];
#pragma unroll
        for (int x = 0; x < MT; ++x) total[x] = 0.f;
        bool go = true;
        for (int slice = 0; slice < slices && go; ++slice) {
            const int buf = slice & 1;
            const bool ok = mbar_wait(&acc_full[buf], (slice >> 1) & 1, 64);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!ok) ring.failed = 1;
            go = __all_sync(0xffffffffu, ok && !ring.failed);  // warp-uniform: the tensor-memory loads are warp-wide
            if (!go) break;
#pragma unroll
            for (int cb = 0; cb < MT / 32; ++cb) {
                uint32_t v[32], w[32];
                tmem_load_32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 2 * MT + cb * 32), v);
                tmem_load_32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 2 * MT + MT + cb * 32), w);
#pragma unroll
                for (int x = 0; x < 32; ++x) total[cb * 32 + x] += __uint_as_float(v[x]) + __uint_as_float(w[x]);
            }
            // this warp has read the accumulators: hand them back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) trinv_arrive(&acc_empty[buf]);
        }
        if (go) {
            const int64_t gi = m0 + q * 32 + lane;
#pragma unroll
            for (int cb = 0; cb < MT / 32; ++cb) {
                float acc[32];
#pragma unroll
                for (int x = 0; x < 32; ++x) acc[x] = total[cb * 32 + x];
                const int64_t gj0 = n0 + cb * 32;
                if (!job.second) {
                    // W^T[gi][gj]: gi is inside the first half (always a row of the matrix), gj is cut at r2
                    float *hi = P.tw_hi + gi * n + gj0, *mid = P.tw_mid + gi * n + gj0, *lo = P.tw_lo + gi * n + gj0;
#pragma unroll
                    for (int x = 0; x < 32; x += 4) {
                        if (gj0 + x < r2) {  // r2 is a multiple of 4: a group is inside or outside as a whole
                            float4 h, c, l;
                            split_tf32_3(acc[x], h.x, c.x, l.x);
                            split_tf32_3(acc[x + 1], h.y, c.y, l.y);
                            split_tf32_3(acc[x + 2], h.z, c.z, l.z);
                            split_tf32_3(acc[x + 3], h.w, c.w, l.w);
                            *reinterpret_cast<float4 *>(hi + x) = h;
                            *reinterpret_cast<float4 *>(mid + x) = c;
                            *reinterpret_cast<float4 *>(lo + x) = l;
                        }
                    }
                } else if (gi < r2) {
                    // X[gi][gj] = -acc: the inverse itself, its split, and the split of its transpose (coalesced across the lanes)
                    float *dst = P.out + gi * n + gj0, *hi = P.out_hi + gi * n + gj0, *mid = P.out_mid + gi * n + gj0, *lo = P.out_lo + gi * n + gj0;
#pragma unroll
                    for (int x = 0; x < 32; x += 4) {
                        const float val[4] = {-acc[x], -acc[x + 1], -acc[x + 2], -acc[x + 3]};
                        float h[4], c[4], l[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            split_tf32_3(val[e], h[e], c[e], l[e]);
                            P.outt_hi[(gj0 + x + e) * n + gi] = h[e];
                            P.outt_mid[(gj0 + x + e) * n + gi] = c[e];
                            P.outt_lo[(gj0 + x + e) * n + gi] = l[e];
                        }
                        *reinterpret_cast<float4 *>(dst + x) = make_float4(val[0], val[1], val[2], val[3]);
                        *reinterpret_cast<float4 *>(hi + x) = make_float4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<float4 *>(mid + x) = make_float4(c[0], c[1], c[2], c[3]);
                        *reinterpret_cast<float4 *>(lo + x) = make_float4(l[0], l[1], l[2], l[3]);
                    }
                }
            }
        }
    }
    const bool failed = tc_ring_teardown(ring, tmem, TRINV_TMEM_COLS);
    if (threadIdx.x == 0 && failed && P.flag) atomicExch(P.flag, -1);
}

// Operand planes after the 64-level of the doubling: T strictly below the diagonal into the lower triangle of tw, and the
// finished 128 x 128 diagonal blocks of Lf (lower triangular) into out / outt with explicit zeros in their other halves.
__global__ void trinv_split_kernel(FactorPlanes p0, FactorPlanes p1) {
    const FactorPlanes P = blockIdx.y ? p1 : p0;
    const int64_t n = P.n, total = n * n;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / n, c = t % n;
        if (c < r) split_tf32_3(P.a[t], P.tw_hi[t], P.tw_mid[t], P.tw_lo[t]);
        if (r / MT == c / MT) {
            split_tf32_3(c <= r ? P.out[t] : 0.f, P.out_hi[t], P.out_mid[t], P.out_lo[t]);
            split_tf32_3(c >= r ? P.out[c * n + r] : 0.f, P.outt_hi[t], P.outt_mid[t], P.outt_lo[t]);
        }
    }
}

static bool factor_maps(FactorMaps *maps, const FactorPlanes &p) {
    float *const out[3] = {p.out_hi, p.out_mid, p.out_lo}, *const outt[3] = {p.outt_hi, p.outt_mid, p.outt_lo}, *const tw[3] = {p.tw_hi, p.tw_mid, p.tw_lo};
    bool ok = true;
    for (int part = 0; part < 3; ++part)
        ok = ok && make_map(&maps->out[part], out[part], p.n, p.n) && make_map(&maps->outt[part], outt[part], p.n, p.n) &&
             make_map(&maps->tw[part], tw[part], p.n, p.n);
    return ok;
}

// Levels b = 128, 256, ... of the doubling for one or two problems whose 128 x 128 diagonal blocks are finished.
int launch_trinv_tc(int count, const FactorPlanes *problems, cudaStream_t stream) {
    static PerDeviceOnce configured;
    const size_t smem = (size_t)TRINV_STAGES * TRINV_STAGE_BYTES + 1024;
    if (configured.run([&] { return cudaFuncSetAttribute(trinv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess; }) != G2D_OK)
        return G2D_ERR_CUDA;
    TrinvJob job;
    int64_t n_max = 0;
    for (int z = 0; z < 2; ++z) {
        job.p[z] = problems[z < count ? z : 0];
        if (!factor_maps(&job.maps[z], job.p[z])) return G2D_ERR_CUDA;
        n_max = job.p[z].n > n_max ? job.p[z].n : n_max;
    }
    trinv_split_kernel<<<dim3(148 * 8, count), 256, 0, stream>>>(job.p[0], job.p[1]);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    for (int64_t b = MT; b < n_max; b *= 2) {
        const int64_t pairs = ceil_div(n_max, 2 * b), tiles = b / MT;
        if (tiles > 65535 || pairs * count > 0x7fffffff) return G2D_ERR_TOO_LARGE;
        job.pairs = (int)pairs;
        job.tiles = (int)tiles;
        job.b = b;
        for (int second = 0; second < 2; ++second) {
            job.second = second;
            trinv_tc_kernel<<<dim3((unsigned)(pairs * count), (unsigned)tiles, (unsigned)tiles), TC_THREADS, smem, stream>>>(job);
            if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        }
    }
    return G2D_OK;
}

// ---- trailing update of the blocked Cholesky factorization ----
// After a group of four 64-row block rows [o, o + kw) is factored, everything above it receives
//     a[r][c] -= sum_{k < kw} a[o + k][r] a[o + k][c],      c <= r < o,
// one 128 x 128 tile per CTA.  Both operands are the same K-major planes pt[r][k] = a[o + k][r] (hi and lo), which
// the panel kernel writes as it finishes a block row.  One CTA owns each target entry and no other kernel touches the
// targets meanwhile, so the result does not depend on scheduling.
// Accuracy.  The tensor cores add each product into the float accumulator with truncation, which biases long sums of
// one sign by about 1e-8 of the sum per term, and the diagonal of this update is a sum of squares, subtracted from pivots
// that a damped, badly conditioned Gram leaves one or two orders of magnitude smaller than the sum.  Two measures keep the
// factors at the accuracy of a float32 LAPACK factorization: the k range is cut into slices of 64 with one accumulator
// each in tensor memory (added up in registers, round to nearest), and the diagonal entries are left out here and
// updated by syrk_diag_kernel with a float64 sum.
constexpr int SYRK_SLICE_CHUNKS = 2;                      // k = 64 per accumulator
constexpr int SYRK_SLICES = SYRK_TC_K / (SYRK_SLICE_CHUNKS * KC);
constexpr uint32_t SYRK_TMEM_COLS = SYRK_SLICES * MT;     // 512: all of tensor memory, one CTA per SM (as its shared memory already requires)
static_assert(SYRK_TMEM_COLS <= 512, "tensor memory holds 512 columns");

struct SyrkJob {
    CUtensorMap hi[2], lo[2];
    float *a[2];
    int64_t n[2];
    int t_lo[2], t_hi[2];  // target tile rows [t_lo, t_hi), with every tile column up to the diagonal
    int chunks[2];         // ceil(kw / 32)
    int *flag[2];
};

__global__ void __launch_bounds__(TC_THREADS) syrk_tc_kernel(const __grid_constant__ SyrkJob job) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) TcRing ring;
    const int z = blockIdx.y;
    const int t_lo = z ? job.t_lo[1] : job.t_lo[0], t_hi = z ? job.t_hi[1] : job.t_hi[0];
    const int64_t first = (int64_t)t_lo * (t_lo + 1) / 2, count = (int64_t)t_hi * (t_hi + 1) / 2 - first;
    if ((int64_t)blockIdx.x >= count) return;
    const int64_t lin = first + blockIdx.x;
    int I2 = (int)((sqrt(8.0 * (double)lin + 1.0) - 1.0) / 2.0);
    while ((int64_t)(I2 + 1) * (I2 + 2) / 2 <= lin) ++I2;
    while ((int64_t)I2 * (I2 + 1) / 2 > lin) --I2;
    const int J2 = (int)(lin - (int64_t)I2 * (I2 + 1) / 2);
    const CUtensorMap *hi = z ? &job.hi[1] : &job.hi[0], *lo = z ? &job.lo[1] : &job.lo[0];
    float *const a = z ? job.a[1] : job.a[0];
    const int64_t n = z ? job.n[1] : job.n[0];
    const int chunks = z ? job.chunks[1] : job.chunks[0];
    int *const flag = z ? job.flag[1] : job.flag[0];
    const int i0 = I2 * MT, j0 = J2 * MT;

    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tmem = tc_ring_setup(ring, SYRK_TMEM_COLS);
    const int slices = (chunks + SYRK_SLICE_CHUNKS - 1) / SYRK_SLICE_CHUNKS;
    if (warp == 0) {
        if (lane == 0)
            tc_ring_produce(ring, smem_base, chunks, [&](int ch, uint32_t dst, uint64_t *bar) {
                tma_load_2d(dst, hi, ch * KC, i0, bar);
                tma_load_2d(dst + TILE_BYTES, lo, ch * KC, i0, bar);
                tma_load_2d(dst + 2 * TILE_BYTES, hi, ch * KC, j0, bar);
                tma_load_2d(dst + 3 * TILE_BYTES, lo, ch * KC, j0, bar);
            });
    } else if (warp == 1) {
        if (lane == 0) {
            // the ring's MMA loop with one accumulator per slice of SYRK_SLICE_CHUNKS chunks
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % STAGES, round = ch / STAGES;
                if (!mbar_wait(&ring.full[stage], round & 1)) {
                    ring.failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(ch / SYRK_SLICE_CHUNKS) * MT;
                const bool first = ch % SYRK_SLICE_CHUNKS == 0;
                const uint32_t a_hi = smem_base + stage * STAGE_BYTES, a_lo = a_hi + TILE_BYTES, b_hi = a_hi + 2 * TILE_BYTES, b_lo = a_hi + 3 * TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < KC / 8; ++ks) {
                    const uint32_t off = ks * 32;
                    umma_tf32(acc, umma_desc(a_hi + off), umma_desc(b_hi + off), IDESC, (first && ks == 0) ? 0u : 1u);
                    umma_tf32(acc, umma_desc(a_lo + off), umma_desc(b_hi + off), IDESC, 1u);
                    umma_tf32(acc, umma_desc(a_hi + off), umma_desc(b_lo + off), IDESC, 1u);
                }
                umma_commit(&ring.empty[stage]);
            }
            umma_commit(&ring.accum);
        }
    } else {
        const int q = warp & 3;
        const bool go = tc_ring_accumulator_ready(ring);
        if (go) {
            const int64_t gi = (int64_t)i0 + q * 32 + lane;  // always a row of the matrix: the targets lie above the group
            for (int cb = 0; cb < MT / 32; ++cb) {
                float sum[32];
#pragma unroll
                for (int x = 0; x < 32; ++x) sum[x] = 0.f;
                for (int sl = 0; sl < slices; ++sl) {
                    uint32_t v[32];
                    tmem_load_32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(sl * MT + cb * 32), v);
#pragma unroll
                    for (int x = 0; x < 32; ++x) sum[x] += __uint_as_float(v[x]);
                }
                const int64_t gj0 = (int64_t)j0 + cb * 32;
                float *dst = a + gi * n + gj0;
#pragma unroll
                for (int x = 0; x < 32; x += 4) {
                    if (gj0 + x <= gi) {  // groups that start right of the diagonal are never read
                        if (gi - (gj0 + x) < 4) {  // the diagonal entry belongs to syrk_diag_kernel
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                if (gj0 + x + c == gi) sum[x + c] = 0.f;
                        }
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + x), "f"(-sum[x]), "f"(-sum[x + 1]),
                                     "f"(-sum[x + 2]), "f"(-sum[x + 3])
                                     : "memory");
                    }
                }
            }
        }
    }
    const bool failed = tc_ring_teardown(ring, tmem, SYRK_TMEM_COLS);
    if (threadIdx.x == 0 && failed && flag) atomicExch(flag, -1);
}

// The diagonal of the same update: a[r][r] -= sum_k p[r][k]^2 with p = hi + lo (the float32 panel value, exactly), the sum
// in float64.  One warp per row.
struct SyrkDiagJob {
    const float *hi[2], *lo[2];
    float *a[2];
    int64_t n[2];
    int64_t r_lo[2], r_hi[2];
    int kw[2];
};
__global__ void syrk_diag_kernel(const SyrkDiagJob job) {
    const int z = blockIdx.y, lane = threadIdx.x & 31;
    const int64_t r_lo = z ? job.r_lo[1] : job.r_lo[0], r_hi = z ? job.r_hi[1] : job.r_hi[0];
    const float *hi = z ? job.hi[1] : job.hi[0], *lo = z ? job.lo[1] : job.lo[0];
    float *a = z ? job.a[1] : job.a[0];
    const int64_t n = z ? job.n[1] : job.n[0];
    const int kw = z ? job.kw[1] : job.kw[0];
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = r_lo + (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < r_hi; r += warps) {
        double sum = 0.0;
        for (int k = lane; k < kw; k += 32) {
            const double p = (double)hi[r * SYRK_TC_K + k] + (double)lo[r * SYRK_TC_K + k];
            sum += p * p;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) a[r * n + r] = (float)((double)a[r * n + r] - sum);
    }
}

bool syrk_tc_maps(SyrkTcMaps *maps, const float *pt_hi, const float *pt_lo, int64_t n) {
    static_assert(sizeof(maps->hi) == sizeof(CUtensorMap), "opaque tensor-map storage has the wrong size");
    return make_map(reinterpret_cast<CUtensorMap *>(maps->hi), pt_hi, n, SYRK_TC_K) &&
           make_map(reinterpret_cast<CUtensorMap *>(maps->lo), pt_lo, n, SYRK_TC_K);
}

int launch_syrk_tc(int count, const SyrkTcTarget *targets, cudaStream_t stream) {
    static PerDeviceOnce configured;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    if (configured.run([&] { return cudaFuncSetAttribute(syrk_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess; }) != G2D_OK)
        return G2D_ERR_CUDA;
    SyrkJob job;
    SyrkDiagJob diag;
    int64_t most = 0, most_rows = 0;
    for (int z = 0; z < 2; ++z) {
        const SyrkTcTarget &t = targets[z < count ? z : 0];
        diag.hi[z] = t.pt_hi; diag.lo[z] = t.pt_lo; diag.a[z] = t.a; diag.n[z] = t.n; diag.kw[z] = t.kw;
        diag.r_lo[z] = (int64_t)t.t_lo * MT;
        diag.r_hi[z] = (int64_t)t.t_hi * MT;  // whole tile rows above the group: every one a row of the matrix
        most_rows = diag.r_hi[z] - diag.r_lo[z] > most_rows ? diag.r_hi[z] - diag.r_lo[z] : most_rows;
        memcpy(&job.hi[z], t.maps->hi, sizeof(CUtensorMap));
        memcpy(&job.lo[z], t.maps->lo, sizeof(CUtensorMap));
        job.a[z] = t.a;
        job.n[z] = t.n;
        job.t_lo[z] = t.t_lo;
        job.t_hi[z] = t.t_hi;
        job.chunks[z] = (t.kw + KC - 1) / KC;
        job.flag[z] = t.flag;
        const int64_t tiles = (int64_t)t.t_hi * (t.t_hi + 1) / 2 - (int64_t)t.t_lo * (t.t_lo + 1) / 2;
        most = tiles > most ? tiles : most;
    }
    if (most <= 0) return G2D_OK;
    if (most > 0x7fffffff) return G2D_ERR_TOO_LARGE;
    syrk_tc_kernel<<<dim3((unsigned)most, count), TC_THREADS, smem, stream>>>(job);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    if (most_rows > 0) {
        int64_t blocks = ceil_div(most_rows * 32, 256);
        syrk_diag_kernel<<<dim3((unsigned)(blocks < 1184 ? blocks : 1184), count), 256, 0, stream>>>(diag);
    }
    return check_launch();
}

}  // namespace g2d
