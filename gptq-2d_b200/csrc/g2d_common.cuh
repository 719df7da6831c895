// Shared definitions of the gptq2d_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "../../include/gptq2d_b200.h"

namespace g2d {

// Geometry of the fused sweep: the matrix is cut into TILE x TILE tiles that are
// swept one tile anti-diagonal at a time; inside a tile, SUB x SUB sub-tiles are
// swept by one warp each, again along anti-diagonals.
constexpr int TILE = 64;
constexpr int SUB = 16;
constexpr int NSUB = TILE / SUB;
constexpr int LD = TILE + 4;  // shared-memory row stride: LD + 1 odd keeps the diagonal walks conflict free

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// IEEE round-to-nearest-even primitives that the compiler may not contract or approximate.
__device__ __forceinline__ float div_rn(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double div_rn(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float rint_even(float a) { return rintf(a); }
__device__ __forceinline__ double rint_even(double a) { return rint(a); }

// (clamp(rint(y / scale + zp), qmin, qmax) - zp) * scale, every step rounded on its own
// (quantizer_int.py:81-83 / :204-205 of the reference).  Comparisons keep NaN like torch.clamp.
template <typename F>
__device__ __forceinline__ F affine_value(F y, F scale, F zp, F qmin, F qmax) {
    F t = rint_even(add_rn(div_rn(y, scale), zp));
    t = t < qmin ? qmin : t;
    t = t > qmax ? qmax : t;
    return mul_rn(sub_rn(t, zp), scale);
}

// The same value with the division done as a product with a precomputed reciprocal `rc` of the scale plus one
// residual correction: q = y rc, q += (y - q s) rc.  With rc within half an ulp of 1 / scale this is the IEEE
// quotient except, rarely, in its last bit, which can change the result only within one ulp of a rounding tie.
// Used inside the fused float sweep, where the exact division sits on the critical path of every stage.
__device__ __forceinline__ float affine_value_rcp(float y, float scale, float zp, float rc, float qmin, float qmax) {
    const float q0 = y * rc;
    const float q = fmaf(fmaf(-q0, scale, y), rc, q0);
    float t = rintf(__fadd_rn(q, zp));
    t = t < qmin ? qmin : t;
    t = t > qmax ? qmax : t;
    return __fmul_rn(__fsub_rn(t, zp), scale);
}
__device__ __forceinline__ double affine_value_rcp(double y, double scale, double zp, double, double qmin, double qmax) {
    return affine_value(y, scale, zp, qmin, qmax);
}

// float -> fp16 / bf16 -> float, round to nearest even (denormals kept).
__device__ __forceinline__ float round_to_half(float f, int half_kind) {
    return half_kind == G2D_BF16 ? __bfloat162float(__float2bfloat16_rn(f)) : __half2float(__float2half_rn(f));
}

// absmax / ((qmax - qmin) / 2) rounded to a 16-bit float through fp32, 0 -> 1 (quantizer_int.py:110-117, :357-363).
template <typename F>
__device__ __forceinline__ F absmax_scale_value(F absmax, F divisor, int half_kind) {
    F s = (F)round_to_half((float)div_rn(absmax, divisor), half_kind);
    return s == (F)0 ? (F)1 : s;
}

// Kernel launches made by this library in this process (read by g2d_launch_count); any host thread may launch.
extern std::atomic<unsigned long long> g_launches;
inline int check_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaPeekAtLastError() == cudaSuccess ? G2D_OK : G2D_ERR_CUDA;
}

// One-time set-up per device (a kernel's opt-in to more than 48 KB of dynamic shared memory), safe when several host
// threads make their first call at the same time: `setup` runs once per device, under a lock, and must return true.
class PerDeviceOnce {
    std::mutex mutex_;
    bool done_[64] = {};

public:
    template <typename Setup>
    int run(Setup &&setup) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return G2D_ERR_CUDA;
        std::lock_guard<std::mutex> lock(mutex_);
        if (!done_[device]) {
            if (!setup()) return G2D_ERR_CUDA;
            done_[device] = true;
        }
        return G2D_OK;
    }
};

// ---- launchers implemented in the .cu files -------------------------------------------------

template <typename F>
struct SweepArgs {
    F *y, *c, *e;  // [batch, m, n] each: Y = X + right feedback (Z where done), C = down feedback, E = errors
    const F *l, *u;
    const int64_t *l_off, *u_off;
    const F *scale, *zero;
    const int64_t *scale_off, *zero_off;
    int64_t srs, scs, zrs, zcs;
    const F *forced;
    F *y_pre;
    F qmin, qmax;
    int kind;
    int64_t batch, m, n;
    int nI, nJ;  // tiles per column / per row
    // float, single matrix, tensor-core updates only (else null): tf32 hi / lo copies of the finished tiles,
    // E transposed ([n, m]) and the completed C ([m, n]), operands of the macro updates
    float *et_hi = nullptr, *et_lo = nullptr, *c_hi = nullptr, *c_lo = nullptr;
    // pipelined schedule only (else null / 0): planes that collect the far feedback apart from Y and C, added when a
    // tile is loaded, and the switch that makes a tile apply the feedback of its two nearest finished neighbours itself
    const F *yf = nullptr, *cf = nullptr;
    int neighbours = 0;
    // pipelined schedule only: the planes through which a tile hands the feedback for its lower and its right neighbour
    // on (the neighbour adds them when it loads); every entry that is read has been written one launch before
    F *yn = nullptr, *cn = nullptr;
};

// fp32 -> tf32 hi (round to nearest) and the fp32 remainder: a = hi + lo exactly, and hi*hi' + lo*hi' + hi*lo' recovers
// the fp32 product to about 2^-21 relative
__device__ __forceinline__ void split_tf32(float a, float &hi, float &lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(a));
    hi = __uint_as_float(h);
    lo = a - hi;
}

// fp32 -> three tf32 values with a = hi + mid + lo exactly (11 + 11 + the last 2 significant bits).  The six products
// hi hi' + hi mid' + mid hi' + mid mid' + hi lo' + lo hi' then carry the fp32 product to about 2^-32: used where the
// 2^-21 of the two-plane split is not enough (the triangular inverse, whose error the condition number amplifies).
__device__ __forceinline__ void split_tf32_3(float a, float &hi, float &mid, float &lo) {
    uint32_t h, m;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(a));
    hi = __uint_as_float(h);
    const float r = a - hi;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(m) : "f"(r));
    mid = __uint_as_float(m);
    lo = r - mid;
}

// Operand planes of the tensor-core macro updates (all float; see g2d_macro_update_tc.cu).
struct TcPlanes {
    float *et_hi, *et_lo, *c_hi, *c_lo;  // written by the tile sweep
    float *l_hi, *l_lo, *ut_hi, *ut_lo;  // written once per sweep from L and U
    int *error_flag;                     // set when a bounded wait inside a kernel ran out
};
// Band updates between tiles on the tensor cores (pipelined schedule; see g2d_band_tc.cu): sources are the tile
// anti-diagonals s0..s1-1, targets t0..t1 (t0 >= s1 + 1), feedback is added into the planes y (right) and c (down).
// With outer_macro > 0 a target is left out when a far update on 128 x 128 macro tiles carries its source instead:
// when its macro anti-diagonal is lag_macro or more past the end of the source's group of outer_macro macro anti-diagonals.
struct BandTcMaps {
    alignas(64) unsigned char bytes[8 * 128];  // tensor maps of the eight operand planes (opaque here)
};
int band_tc_prepare(BandTcMaps *maps, const TcPlanes &planes, int64_t m, int64_t n);
int launch_band_tc(const BandTcMaps *maps, float *y, float *c, int64_t m, int64_t n, int s0, int s1, int t0, int t1, int outer_macro,
                   int lag_macro, int *error_flag, cudaStream_t stream);
int tc_prepare_operands(const float *l, const float *u, int64_t m, int64_t n, const TcPlanes &planes, cudaStream_t stream);
struct MacroTcMaps {
    alignas(64) unsigned char bytes[8 * 128];  // tensor maps of the eight operand planes with 128-row boxes (opaque here)
};
int macro_tc_prepare(MacroTcMaps *maps, const TcPlanes &planes, int64_t m, int64_t n);
int launch_macro_update_tc(const MacroTcMaps *maps, const TcPlanes &planes, float *y, float *c, int64_t m, int64_t n, int s0, int s1, int s_end,
                           cudaStream_t stream, int t_first = 0, int stages = 3);

// One problem of the tensor-core triangular inverse of the factor preparation (all [n][n] float; see g2d_factors_tc.cu).
struct FactorPlanes {
    const float *a;            // Cholesky factor T in its lower triangle
    float *out;                // the inverse being built
    // every operand as three tf32 planes hi + mid + lo = the float32 value exactly (see split_tf32_3):
    float *out_hi, *out_mid, *out_lo;      // the inverse
    float *outt_hi, *outt_mid, *outt_lo;   // its transpose
    float *tw_hi, *tw_mid, *tw_lo;         // lower triangle: T; upper triangle: the transposed intermediate product
    int64_t n;
    int *flag;                 // receives -1 when a bounded wait inside a kernel ran out (may be null)
};
int launch_trinv_tc(int count, const FactorPlanes *problems, cudaStream_t stream);

// Tensor-core trailing update of the blocked Cholesky factorization (see g2d_factors_tc.cu).  pt planes are
// [n][SYRK_TC_K] float: pt[r][k] = a[o + k][r] for the group of block rows that starts at row o.
constexpr int SYRK_TC_K = 256;
struct SyrkTcMaps {
    alignas(64) unsigned char hi[128], lo[128];  // tensor maps of the hi and lo planes (opaque here)
};
struct SyrkTcTarget {
    const SyrkTcMaps *maps;
    const float *pt_hi, *pt_lo;  // the planes the maps describe
    float *a;
    int64_t n;
    int t_lo, t_hi;  // target 128-row tile rows [t_lo, t_hi), tile columns up to the diagonal
    int kw;          // rows of the group (<= SYRK_TC_K)
    int *flag;
};
bool syrk_tc_maps(SyrkTcMaps *maps, const float *pt_hi, const float *pt_lo, int64_t n);
int launch_syrk_tc(int count, const SyrkTcTarget *targets, cudaStream_t stream);

// Trellis (Viterbi) search of `rows` sequences (see g2d_trellis.cu); `codes` optional packed paths, code bytes apart.
int64_t trellis_code_bytes(int T, int L, int K, int V, int tail_biting);
size_t trellis_scratch_bytes(int dtype, int64_t rows, int T, int L, int K, int V);
// An optional index of the code table: its distinct rows ([count, V], in the table's dtype) and, per state, the number of
// its row among them.  Tables with few distinct rows are searched from shared memory with it (same results).
struct TrellisIndex {
    const void *distinct;
    const uint16_t *ids;
    int count;
};
int launch_trellis(int dtype, int64_t rows, int T, const void *x, const void *table, int L, int K, int V, int tail, const void *scale,
                   void *out, int64_t *states, void *workspace, uint8_t *codes, cudaStream_t st, const TrellisIndex *index = nullptr);

template <typename F>
int launch_tile_sweep(const SweepArgs<F> &args, int S, cudaStream_t stream, int parity = 0);

enum BandMode { BAND_TILE = 0, BAND_PLAIN = 1, BAND_GENERAL = 2 };

template <typename F>
struct BandArgs {
    F *y, *c;
    const F *e, *l, *u;
    const int64_t *l_off, *u_off;
    int64_t batch, m, n;
    int P, Q;                 // stage(i, j) = i / P + j / Q
    int64_t s0, s1, s_end;    // sources s0..s1-1, targets s1..s_end-1
    int down_into_y;          // also add the down product into Y (the generic path keeps Y live)
    int mode;                 // BandMode
    int filter;               // tile mode only: 0 none, 1 sources with even tile row and column only, 2 targets with odd tile row and column only
    const int32_t *skew = nullptr;  // general mode only: batch b takes the stages s0 - skew[b], s1 - skew[b], s_end - skew[b]
};

template <typename F>
int launch_band_update(const BandArgs<F> &args, cudaStream_t stream);

// skew (device, one int per batch, may be null): batch b works at stage s - skew[b] (slabs of an N-factor sweep);
// z_stride: values of z per batch (0: exactly the stage's d p q)
template <typename F>
int launch_stage_push(const g2d_stage_desc &d, const F *z, int64_t s, int64_t s1, cudaStream_t stream, const int32_t *skew = nullptr,
                      int64_t z_stride = 0);

}  // namespace g2d
