// Hessian-factor accumulation on the tensor cores (float only): H += alpha X^T X for a batch of activations
// X [k samples, n channels], the step before ldl_of_inverse in a quantization pipeline.  The reference takes its
// Hessian factors from the caller (demo.ipynb:103-106 forms them with a plain matrix product), so this entry has no
// counterpart there.
//
// X^T is first written as K-major tf32 hi / lo planes [n][k] (one transposing pass), then every 128 x 128 tile of the
// lower triangle of H is one CTA of the same pipeline as the other tensor-core kernels: TMA into a three-stage ring,
// tcgen05.mma kind::tf32 with the 3xTF32 split (hi hi + lo hi + hi lo) into tensor memory, and an epilogue that adds
// alpha times the accumulator to the lower triangle of H, slice of k by slice of k; a last pass mirrors the lower triangle
// into the upper one (H is symmetric on entry and stays so bit for bit).  Every entry of H has one owner, so the result does not depend on scheduling.
#include "g2d_tc.cuh"

namespace g2d {

// X [k][n] -> planes [n][kp], kp = k rounded up to a multiple of 4 (a TMA stride must be a multiple of 16 bytes); the
// padding columns are zero
__global__ void gram_split_transposed_kernel(const float *__restrict__ x, int64_t k, int64_t n, int64_t kp, float *__restrict__ hi,
                                             float *__restrict__ lo) {
    __shared__ float tile[32][33];
    const int64_t tiles_s = ceil_div(kp, (int64_t)32), tiles_j = ceil_div(n, (int64_t)32);
    for (int64_t b = blockIdx.x; b < tiles_s * tiles_j; b += gridDim.x) {
        const int64_t s0 = (b / tiles_j) * 32, j0 = (b % tiles_j) * 32;  // source block: samples s, channels j
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t s = s0 + r, j = j0 + threadIdx.x;
            tile[r][threadIdx.x] = (s < k && j < n) ? x[s * n + j] : 0.f;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t j = j0 + r, s = s0 + threadIdx.x;
            if (j < n && s < kp) {
                float h, l;
                split_tf32(tile[threadIdx.x][r], h, l);
                hi[j * kp + s] = h;
                lo[j * kp + s] = l;
            }
        }
        __syncthreads();
    }
}

struct GramJob {
    CUtensorMap hi, lo;
    float *h;
    int64_t n;
    int chunks;
    float alpha;
    int *flag;
};

// The tensor cores add into their fp32 accumulator with truncation, which biases a long sum of same-sign terms (the
// diagonal of a Gram matrix is a sum of squares): measured 9e-5 relative over k = 8192 in one accumulator.  So the k
// range is cut into slices of SLICE chunks; each slice is accumulated in tensor memory and then added to H in global
// memory with round-to-nearest reductions.  Two accumulators alternate, so the epilogue of a slice overlaps the MMAs
// of the next.
constexpr int SLICE = 4;  // 128 samples per slice
constexpr uint32_t GRAM_TMEM_COLS = 256;

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(TC_THREADS) gram_tc_kernel(const __grid_constant__ GramJob job) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    // tile (I2, J2), J2 <= I2, from the linear index
    const int64_t lin = blockIdx.x;
    int I2 = (int)((sqrt(8.0 * (double)lin + 1.0) - 1.0) / 2.0);
    while ((int64_t)(I2 + 1) * (I2 + 2) / 2 <= lin) ++I2;
    while ((int64_t)I2 * (I2 + 1) / 2 > lin) --I2;
    const int J2 = (int)(lin - (int64_t)I2 * (I2 + 1) / 2);
    const int i0 = I2 * MT, j0 = J2 * MT;
    const int64_t n = job.n;
    const int chunks = job.chunks, slices = (chunks + SLICE - 1) / SLICE;

    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);  // one arrival per epilogue warp
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(GRAM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % STAGES, round = ch / STAGES;
                if (round > 0 && !mbar_wait(&empty_bar[stage], (round - 1) & 1)) { failed = 1; break; }
                const uint32_t dst = smem_base + stage * STAGE_BYTES;
                mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
                tma_load_2d(dst, &job.hi, ch * KC, i0, &full_bar[stage]);
                tma_load_2d(dst + TILE_BYTES, &job.lo, ch * KC, i0, &full_bar[stage]);
                tma_load_2d(dst + 2 * TILE_BYTES, &job.hi, ch * KC, j0, &full_bar[stage]);
                tma_load_2d(dst + 3 * TILE_BYTES, &job.lo, ch * KC, j0, &full_bar[stage]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int ch = 0; ch < chunks; ++ch) {
                const int stage = ch % STAGES, round = ch / STAGES;
                const int slice = ch / SLICE, buf = slice & 1;
                const bool opens = ch % SLICE == 0, closes = ch % SLICE == SLICE - 1 || ch == chunks - 1;
                // the accumulator must have been read out by the epilogue of the slice two before
                if (opens && slice >= 2 && !mbar_wait(&acc_empty[buf], ((slice >> 1) - 1) & 1)) { failed = 1; break; }
                if (!mbar_wait(&full_bar[stage], round & 1)) { failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem + (uint32_t)(buf * MT);
                const uint32_t a_hi = smem_base + stage * STAGE_BYTES, a_lo = a_hi + TILE_BYTES, b_hi = a_hi + 2 * TILE_BYTES, b_lo = a_hi + 3 * TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < KC / 8; ++ks) {
                    const uint32_t off = ks * 32;  // 8 tf32 values = 32 bytes along the swizzled row
                    umma_tf32(d, umma_desc(a_hi + off), umma_desc(b_hi + off), IDESC, (opens && ks == 0) ? 0u : 1u);
                    umma_tf32(d, umma_desc(a_lo + off), umma_desc(b_hi + off), IDESC, 1u);
                    umma_tf32(d, umma_desc(a_hi + off), umma_desc(b_lo + off), IDESC, 1u);
                }
                umma_commit(&empty_bar[stage]);            // arrives when the MMAs above have read the stage
                if (closes) umma_commit(&acc_full[buf]);   // arrives when the slice is complete in tensor memory
            }
        }
    } else {
        // epilogue warps: lanes 32 q .. 32 q + 31 of tensor memory, q = warp % 4; one accumulator row per thread
        const int q = warp & 3;
        const int64_t gi = (int64_t)i0 + q * 32 + lane;
        for (int slice = 0; slice < slices; ++slice) {
            const int buf = slice & 1;
            const bool ok = mbar_wait(&acc_full[buf], (slice >> 1) & 1, 64);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!ok) failed = 1;
            if (!__all_sync(0xffffffffu, ok && !failed)) break;  // warp-uniform: the tensor-memory loads are warp-wide
            for (int cb = 0; cb < MT / 32; ++cb) {
                uint32_t v[32];
                tmem_load_32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * MT + cb * 32), v);
                const int64_t gj0 = (int64_t)j0 + cb * 32;
                if (gi < n) {
                    // only the lower triangle is accumulated here; a pass at the end copies it to the upper one
                    float *dst = job.h + gi * n + gj0;
                    if (I2 != J2) {
#pragma unroll
                        for (int x = 0; x < 32; x += 4) {
                            if (gj0 + x < n) {  // n is a multiple of 4: a group is inside or outside as a whole
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + x), "f"(job.alpha * __uint_as_float(v[x])),
                                             "f"(job.alpha * __uint_as_float(v[x + 1])), "f"(job.alpha * __uint_as_float(v[x + 2])),
                                             "f"(job.alpha * __uint_as_float(v[x + 3]))
                                             : "memory");
                            }
                        }
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x) {
                            if (gj0 + x <= gi)
                                asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + x), "f"(job.alpha * __uint_as_float(v[x])) : "memory");
                        }
                    }
                }
            }
            // this warp has read the accumulator: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        if (failed) {
            // give outstanding loads and MMAs a bounded chance to land before the memory they target is released
            if (lane == 0) mbar_wait(&acc_full[((slices - 1) & 1)], ((slices - 1) >> 1) & 1);
            __syncwarp();
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(GRAM_TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && job.flag) atomicExch(job.flag, -1);
}

// H[j][i] = H[i][j] for j < i: the upper triangle from the lower one, 32 x 32 blocks through shared memory
__global__ void gram_mirror_kernel(float *__restrict__ h, int64_t n) {
    __shared__ float tile[32][33];
    const int64_t tiles = ceil_div(n, (int64_t)32);
    for (int64_t b = blockIdx.x; b < tiles * tiles; b += gridDim.x) {
        const int64_t bi = b / tiles, bj = b % tiles;
        if (bj > bi) continue;  // source blocks of the lower triangle, the diagonal blocks included
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t i = bi * 32 + r, j = bj * 32 + threadIdx.x;
            tile[r][threadIdx.x] = (i < n && j < n) ? h[i * n + j] : 0.f;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t j = bj * 32 + r, i = bi * 32 + threadIdx.x;  // target (j, i), strictly above the diagonal
            if (i < n && j < n && j < i) h[j * n + i] = tile[threadIdx.x][r];
        }
        __syncthreads();
    }
}

}  // namespace g2d

using namespace g2d;

// samples rounded up to a multiple of 4 (16-byte strides), at least one k chunk
static int64_t gram_padded(int64_t k) { return k < 32 ? 32 : (k + 3) / 4 * 4; }

static size_t gram_bytes(int64_t n, int64_t k) {
    const size_t kp = (size_t)gram_padded(k);
    return (2 * (size_t)n * kp * sizeof(float) + 255) & ~(size_t)255;
}

extern "C" int g2d_gram_workspace_bytes(int64_t n, int64_t k, size_t *bytes) {
    if (n < 0 || k < 0 || !bytes) return G2D_ERR_BAD_ARGUMENT;
    *bytes = gram_bytes(n, k);
    return G2D_OK;
}

extern "C" int g2d_gram_accumulate(int64_t n, int64_t k, const float *x, float alpha, float *h, int32_t *status_flag, void *workspace,
                                   size_t workspace_bytes, void *stream) {
    if (n < 0 || k < 0) return G2D_ERR_BAD_ARGUMENT;
    if (n == 0 || k == 0) return G2D_OK;
    if (!x || !h || n % 4 != 0 || ((uintptr_t)h & 15) != 0) return G2D_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < gram_bytes(n, k) || ((uintptr_t)workspace & 255) != 0) return G2D_ERR_WORKSPACE;
    const int64_t kp = gram_padded(k), tiles = ceil_div(n, (int64_t)MT);
    if (tiles * (tiles + 1) / 2 > 0x7fffffff || kp > 0x7fffffff) return G2D_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    static PerDeviceOnce configured;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    if (configured.run([&] { return cudaFuncSetAttribute(gram_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess; }) != G2D_OK)
        return G2D_ERR_CUDA;
    float *hi = (float *)workspace, *lo = hi + n * kp;
    gram_split_transposed_kernel<<<148 * 8, dim3(32, 8), 0, st>>>(x, k, n, kp, hi, lo);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    GramJob job;
    if (!make_map(&job.hi, hi, n, kp) || !make_map(&job.lo, lo, n, kp)) return G2D_ERR_CUDA;
    job.h = h;
    job.n = n;
    job.chunks = (int)ceil_div(kp, (int64_t)KC);
    job.alpha = alpha;
    job.flag = status_flag;
    gram_tc_kernel<<<(unsigned)(tiles * (tiles + 1) / 2), TC_THREADS, smem, st>>>(job);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    gram_mirror_kernel<<<148 * 8, dim3(32, 8), 0, st>>>(h, n);
    return check_launch();
}
