// Building blocks shared by the tensor-core kernels: mbarrier, TMA and tcgen05 wrappers, the shared-memory operand
// descriptor of a K-major 128 x 32 fp32 tile with 128-byte swizzle, and the host-side tensor-map encoder.
#pragma once
#include <cuda.h>

#include "g2d_common.cuh"

namespace g2d {

constexpr int MT = 128;                    // macro tile edge
constexpr int KC = 32;                     // k per chunk: 32 floats = one 128-byte swizzle row
constexpr int TILE_BYTES = MT * KC * 4;    // 16 KB
constexpr int STAGE_BYTES = 4 * TILE_BYTES;
constexpr int STAGES = 3;
constexpr int TC_THREADS = 192;
constexpr uint32_t TMEM_COLS = 256;
constexpr long long WAIT_CYCLES = 2000000000LL;  // about a second

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// false on time-out.  Between polls the warp sleeps for `nap` nanoseconds: these kernels share SMs with the tile sweep,
// whose two working warps should not lose issue slots to a spinning neighbour.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned nap = 32) {
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > WAIT_CYCLES) return false;
        __nanosleep(nap);
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// K-major operand tile of 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);   // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
    d |= (uint64_t)1 << 46;                       // descriptor version
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
// D fp32, A and B tf32, both K-major, M = 128, N = 128
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(MT >> 3) << 17) | ((uint32_t)(MT >> 4) << 24);

// 32 consecutive accumulator columns of this warp's 32 tensor-memory lanes (one row per thread)
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&v)[32]) {
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
}

// ---- one-accumulator pipeline: C[128 x 128] = sum over k chunks of A[128 x 32] B[128 x 32]^T, 3xTF32 ----
// Shared state of a CTA of TC_THREADS threads: warp 0 loads, warp 1 issues the MMAs, warps 2-5 read the accumulator.
struct TcRing {
    uint64_t full[STAGES], empty[STAGES], accum;
    uint32_t tmem_slot;
    int failed;
};

// All threads: barriers, tensor-memory allocation of `cols` columns (by warp 1); returns the accumulator's address.
__device__ __forceinline__ uint32_t tc_ring_setup(TcRing &ring, uint32_t cols) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ring.full[s], 1);
            mbar_init(&ring.empty[s], 1);
        }
        mbar_init(&ring.accum, 1);
        ring.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ring.tmem_slot)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return ring.tmem_slot;
}

// One thread: for every chunk, wait for its stage to be free and call load(chunk, destination, barrier), which must
// issue TMA loads of STAGE_BYTES in total (A_hi, A_lo, B_hi, B_lo tiles, TILE_BYTES apart).
template <typename Load>
__device__ __forceinline__ void tc_ring_produce(TcRing &ring, uint32_t smem_base, int chunks, Load load) {
    for (int ch = 0; ch < chunks; ++ch) {
        const int stage = ch % STAGES, round = ch / STAGES;
        if (round > 0 && !mbar_wait(&ring.empty[stage], (round - 1) & 1)) {
            ring.failed = 1;
            break;
        }
        mbar_expect_tx(&ring.full[stage], STAGE_BYTES);
        load(ch, smem_base + stage * STAGE_BYTES, &ring.full[stage]);
    }
}

// One thread: the MMAs of every chunk into the accumulator at `tmem`, then the commit that the epilogue waits for.
__device__ __forceinline__ void tc_ring_mma(TcRing &ring, uint32_t smem_base, uint32_t tmem, int chunks) {
    for (int ch = 0; ch < chunks; ++ch) {
        const int stage = ch % STAGES, round = ch / STAGES;
        if (!mbar_wait(&ring.full[stage], round & 1)) {
            ring.failed = 1;
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_hi = smem_base + stage * STAGE_BYTES, a_lo = a_hi + TILE_BYTES, b_hi = a_hi + 2 * TILE_BYTES, b_lo = a_hi + 3 * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < KC / 8; ++ks) {
            const uint32_t off = ks * 32;  // 8 tf32 values = 32 bytes along the swizzled row
            umma_tf32(tmem, umma_desc(a_hi + off), umma_desc(b_hi + off), IDESC, (ch == 0 && ks == 0) ? 0u : 1u);
            umma_tf32(tmem, umma_desc(a_lo + off), umma_desc(b_hi + off), IDESC, 1u);
            umma_tf32(tmem, umma_desc(a_hi + off), umma_desc(b_lo + off), IDESC, 1u);
        }
        umma_commit(&ring.empty[stage]);  // arrives when the MMAs above have read the stage
    }
    umma_commit(&ring.accum);             // arrives when every MMA issued so far has completed
}

// Epilogue warps: wait for the accumulator; false (for the whole warp) if any wait of the CTA ran out.
__device__ __forceinline__ bool tc_ring_accumulator_ready(TcRing &ring) {
    const bool ok = mbar_wait(&ring.accum, 0, 256);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!ok) ring.failed = 1;
    return __all_sync(0xffffffffu, ok && !ring.failed);  // warp-uniform: the tensor-memory loads are warp-wide
}

// All threads: release tensor memory; returns whether a wait ran out (meaningful in every thread).
__device__ __forceinline__ bool tc_ring_teardown(TcRing &ring, uint32_t tmem, uint32_t cols) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == 1) {
        if (ring.failed) {
            // give outstanding loads and MMAs a bounded chance to land before the memory they target is released
            if ((threadIdx.x & 31) == 0) mbar_wait(&ring.accum, 0);
            __syncwarp();
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(cols) : "memory");
    }
    return ring.failed != 0;
}

// ---- host side: tensor maps ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// row-major fp32 matrix [rows][cols]; boxes of box_rows rows x 32 columns, 128-byte swizzle, zero fill outside
static bool make_map(CUtensorMap *map, const float *base, int64_t rows, int64_t cols, int box_rows = MT) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
    const cuuint32_t box[2] = {KC, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


}  // namespace g2d
