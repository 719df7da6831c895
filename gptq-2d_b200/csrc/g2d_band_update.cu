// Band update: apply the errors of the stages s0..s1-1 to the stages s1..s_end-1 as dense products.
//
//     down :  C[i, j] += sum_k L[i, k] E[k, j]   over the sources (k, j) of the band
//     right:  Y[i, j] += sum_k C[i, k] U[k, j]   over the sources (i, k) of the band
//
// with stage(i, j) = i / P + j / Q.  This is the work of _repack_errors_kernel + _flush_down_kernel +
// _flush_right_kernel of the reference (gptq_2d.py:632-1057).  The errors stay in their natural
// [m, n] layout and the band is selected by masks while the operands are staged in shared memory, so
// there is no repacking pass.  In tile mode (P = Q = TILE, used by the fused sweep) stages are tile
// anti-diagonals, every operand block is either wholly inside or wholly outside the band and the
// k range of a target tile is exact; the plain (P = Q = 1) and general modes serve the generic path.
//
// One CTA of 64 threads owns one 64 x 64 target tile; each thread accumulates 8 x 8 outputs in
// registers, operands are staged 16 k at a time.
#include "g2d_common.cuh"

namespace g2d {

constexpr int BT = 64;       // target tile edge
constexpr int BK = 16;       // k chunk
constexpr int BTH = 64;      // threads per CTA
constexpr int BLD = BT + 4;  // shared row stride of the staged operands

// Thread (ty, tx) of the 8 x 8 thread grid owns rows ty*4 + {0..3} and 32 + ty*4 + {0..3} (columns likewise with tx),
// so that its shared-memory reads are two 16-byte vectors that never collide with its neighbours'.
__device__ __forceinline__ int own(int t, int x) { return x < 4 ? t * 4 + x : 32 + t * 4 + (x - 4); }

template <typename F, int MODE>
struct BandGeom {
    int P, Q;
    int64_t s0, s1, s_end;
    __device__ __forceinline__ int64_t stage(int64_t i, int64_t j) const {
        if (MODE == BAND_TILE) return (i / TILE) + (j / TILE);
        if (MODE == BAND_PLAIN) return i + j;
        return i / P + j / Q;
    }
    __device__ __forceinline__ int64_t brow(int64_t i) const { return MODE == BAND_TILE ? i / TILE : (MODE == BAND_PLAIN ? i : i / P); }
    __device__ __forceinline__ int64_t bcol(int64_t j) const { return MODE == BAND_TILE ? j / TILE : (MODE == BAND_PLAIN ? j : j / Q); }
};

// acc[8][8] += A[i0.., k_lo..k_hi) * B[k_lo..k_hi), j0..) with element masks:
//   DOWN : A = L[i, k] where brow(k) < brow(i);       B = E[k, j] where stage(k, j) in [s0, s1)
//   RIGHT: A = C[i, k] where stage(i, k) in [s0, s1);  B = U[k, j] where bcol(k) < bcol(j)
template <typename F, int MODE, bool DOWN>
__device__ __forceinline__ void band_product(F (&acc)[8][8], const F *__restrict__ A, int64_t lda, const F *__restrict__ B,
                                             int64_t ldb, int64_t i0, int64_t j0, int64_t rows, int64_t cols,
                                             int64_t k_lo, int64_t k_hi, const BandGeom<F, MODE> &g, F *As, F *Bs) {
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
    for (int64_t k0 = k_lo; k0 < k_hi; k0 += BK) {
        // stage A transposed (As[kk][row]) and B (Bs[kk][col])
        for (int idx = tid; idx < BT * BK; idx += BTH) {
            const int row = idx / BK, kk = idx % BK;
            const int64_t i = i0 + row, k = k0 + kk;
            bool ok = i < rows && k < k_hi;
            if (MODE != BAND_TILE && ok) ok = DOWN ? g.brow(k) < g.brow(i) : (g.stage(i, k) >= g.s0 && g.stage(i, k) < g.s1);
            As[kk * BLD + row] = ok ? A[i * lda + k] : (F)0;
        }
        for (int idx = tid; idx < BT * BK; idx += BTH) {
            const int kk = idx / BT, col = idx % BT;
            const int64_t k = k0 + kk, j = j0 + col;
            bool ok = j < cols && k < k_hi;
            if (MODE != BAND_TILE && ok) ok = DOWN ? (g.stage(k, j) >= g.s0 && g.stage(k, j) < g.s1) : g.bcol(k) < g.bcol(j);
            Bs[kk * BLD + col] = ok ? B[k * ldb + j] : (F)0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            F a[8], b[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) a[x] = As[kk * BLD + own(ty, x)];
#pragma unroll
            for (int y = 0; y < 8; ++y) b[y] = Bs[kk * BLD + own(tx, y)];
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] += a[x] * b[y];
        }
        __syncthreads();
    }
}

template <typename F>
__device__ __forceinline__ void ld4(const F *p, F (&v)[4]);
template <>
__device__ __forceinline__ void ld4<float>(const float *p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void ld4<double>(const double *p, double (&v)[4]) {
    const double2 a = *reinterpret_cast<const double2 *>(p), b = *reinterpret_cast<const double2 *>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename F>
__device__ __forceinline__ void st4(F *p, const F (&v)[4]);
template <>
__device__ __forceinline__ void st4<float>(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void st4<double>(double *p, const double (&v)[4]) {
    *reinterpret_cast<double2 *>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2 *>(p + 2) = make_double2(v[2], v[3]);
}

// Interior tiles in tile mode: no masks, 16-byte vector loads, the next k chunk travels from global memory to
// registers while the current one is multiplied out of shared memory (two shared buffers, one barrier per chunk).
// Thread (ty, tx) owns rows ty*4 + {0..3} and 32 + ty*4 + {0..3}, columns tx*4 + {0..3} and 32 + tx*4 + {0..3}:
// acc[x][y] with x, y < 4 the first group and >= 4 the second.
template <typename F>
__device__ __forceinline__ void band_product_fast(F (&acc)[8][8], const F *__restrict__ A, int64_t lda, const F *__restrict__ B,
                                                  int64_t ldb, int64_t i0, int64_t j0, int64_t k_lo, int64_t k_hi, F *As, F *Bs) {
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
    constexpr int BUF = BK * BLD;
    F ra[4][4], rb[4][4];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int id = t * BTH + tid;
            ld4(A + (i0 + (id >> 2)) * lda + k0 + (id & 3) * 4, ra[t]);
            ld4(B + (k0 + (id >> 4)) * ldb + j0 + (id & 15) * 4, rb[t]);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int id = t * BTH + tid;
            const int row = id >> 2, kq = (id & 3) * 4;
#pragma unroll
            for (int x = 0; x < 4; ++x) As[buf * BUF + (kq + x) * BLD + row] = ra[t][x];
            st4(Bs + buf * BUF + (id >> 4) * BLD + (id & 15) * 4, rb[t]);
        }
    };
    fetch(k_lo);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int64_t k0 = k_lo; k0 < k_hi; k0 += BK) {
        const bool more = k0 + BK < k_hi;
        if (more) fetch(k0 + BK);
        const F *as = As + buf * BUF, *bs = Bs + buf * BUF;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            F a[8], b[8];
            F t4[4];
            ld4(as + kk * BLD + ty * 4, t4);
#pragma unroll
            for (int x = 0; x < 4; ++x) a[x] = t4[x];
            ld4(as + kk * BLD + 32 + ty * 4, t4);
#pragma unroll
            for (int x = 0; x < 4; ++x) a[4 + x] = t4[x];
            ld4(bs + kk * BLD + tx * 4, t4);
#pragma unroll
            for (int x = 0; x < 4; ++x) b[x] = t4[x];
            ld4(bs + kk * BLD + 32 + tx * 4, t4);
#pragma unroll
            for (int x = 0; x < 4; ++x) b[4 + x] = t4[x];
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] += a[x] * b[y];
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
}

template <typename F, int MODE>
__global__ void __launch_bounds__(BTH) band_update_kernel(BandArgs<F> P, int nTI, int nTJ, int a_lo) {
    __shared__ __align__(16) F As[2 * BK * BLD];
    __shared__ __align__(16) F Bs[2 * BK * BLD];
    // blockIdx.y selects a target tile anti-diagonal, blockIdx.x a tile on it
    const int A = a_lo + (int)blockIdx.y;
    const int ti_lo = max(0, A - nTJ + 1), ti_hi = min(A + 1, nTI);
    const int TI = ti_lo + (int)blockIdx.x;
    if (TI >= ti_hi) return;
    const int TJ = A - TI;
    const int64_t m = P.m, n = P.n;
    const int64_t i0 = (int64_t)TI * BT, j0 = (int64_t)TJ * BT;
    const int64_t i1 = min(i0 + BT, m) - 1, j1 = min(j0 + BT, n) - 1;  // last row / column of the tile
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;

    for (int64_t batch = blockIdx.z; batch < P.batch; batch += gridDim.z) {
        // the band of this batch: the same for every batch unless the batches are the skewed slabs of an N-factor sweep
        const int64_t behind = (MODE == BAND_GENERAL && P.skew != nullptr) ? P.skew[batch] : 0;
        const int64_t s0 = P.s0 - behind, s1 = P.s1 - behind, s_end = P.s_end - behind;
        BandGeom<F, MODE> g{P.P, P.Q, s0, s1, s_end};
        // does the tile hold any target?
        if (g.stage(i1, j1) < s1 || g.stage(i0, j0) >= s_end) continue;
        // k ranges: block rows (down) / block columns (right) that hold sources for this tile
        const int64_t PP = MODE == BAND_TILE ? TILE : (MODE == BAND_PLAIN ? 1 : P.P);
        const int64_t QQ = MODE == BAND_TILE ? TILE : (MODE == BAND_PLAIN ? 1 : P.Q);
        int64_t dk_lo = (s0 - g.bcol(j1)) * PP, dk_hi = (s1 - g.bcol(j0)) * PP;
        dk_lo = max(dk_lo, (int64_t)0);
        dk_hi = min(min(dk_hi, m), g.brow(i1) * PP);  // sources lie in block rows above the targets
        int64_t rk_lo = (s0 - g.brow(i1)) * QQ, rk_hi = (s1 - g.brow(i0)) * QQ;
        rk_lo = max(rk_lo, (int64_t)0);
        rk_hi = min(min(rk_hi, n), g.bcol(j1) * QQ);
        if (MODE == BAND_TILE && P.filter == 2 && !((TI & 1) && (TJ & 1))) continue;
        if (MODE == BAND_TILE && P.filter == 1) {
            // single-stage use: the down source is tile (dk_lo / 64, TJ), the right source tile (TI, rk_lo / 64)
            if ((TJ & 1) || ((dk_lo / TILE) & 1)) dk_hi = dk_lo;
            if ((TI & 1) || ((rk_lo / TILE) & 1)) rk_hi = rk_lo;
        }
        F *yg = P.y + batch * m * n, *cg = P.c + batch * m * n;
        const F *eg = P.e + batch * m * n;
        const F *lg = P.l + (P.l_off ? P.l_off[batch] : 0);
        const F *ug = P.u + (P.u_off ? P.u_off[batch] : 0);
        // interior tiles of the fused sweep take the vectorised, double-buffered product
        const bool fast = MODE == BAND_TILE && i0 + BT <= m && j0 + BT <= n && m % 4 == 0 && n % 4 == 0 &&
                          ((reinterpret_cast<uintptr_t>(yg) | reinterpret_cast<uintptr_t>(cg) | reinterpret_cast<uintptr_t>(eg) |
                            reinterpret_cast<uintptr_t>(lg) | reinterpret_cast<uintptr_t>(ug)) % (4 * sizeof(F)) == 0);
        F acc[8][8];
        if (dk_lo < dk_hi) {
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] = (F)0;
            if (fast) band_product_fast<F>(acc, lg, m, eg, n, i0, j0, dk_lo, dk_hi, As, Bs);
            else band_product<F, MODE, true>(acc, lg, m, eg, n, i0, j0, m, n, dk_lo, dk_hi, g, As, Bs);
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const int64_t i = i0 + own(ty, x);
#pragma unroll
                for (int y = 0; y < 8; ++y) {
                    const int64_t j = j0 + own(tx, y);
                    if (i < m && j < n) {
                        const int64_t st = g.stage(i, j);
                        if (st >= s1 && st < s_end) {
                            cg[i * n + j] += acc[x][y];
                            if (P.down_into_y) yg[i * n + j] += acc[x][y];
                        }
                    }
                }
            }
        }
        if (rk_lo < rk_hi) {
            // reads C only on sources of the band, which no CTA of this launch writes
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] = (F)0;
            if (fast) band_product_fast<F>(acc, cg, n, ug, n, i0, j0, rk_lo, rk_hi, As, Bs);
            else band_product<F, MODE, false>(acc, cg, n, ug, n, i0, j0, m, n, rk_lo, rk_hi, g, As, Bs);
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const int64_t i = i0 + own(ty, x);
#pragma unroll
                for (int y = 0; y < 8; ++y) {
                    const int64_t j = j0 + own(tx, y);
                    if (i < m && j < n) {
                        const int64_t st = g.stage(i, j);
                        if (st >= s1 && st < s_end) yg[i * n + j] += acc[x][y];
                    }
                }
            }
        }
    }
}

template <typename F>
int launch_band_update(const BandArgs<F> &args, cudaStream_t stream) {
    const int nTI = (int)ceil_div(args.m, BT), nTJ = (int)ceil_div(args.n, BT);
    int a_lo = 0, a_hi = nTI + nTJ - 2;  // target tile anti-diagonals (inclusive)
    if (args.mode == BAND_TILE) {
        a_lo = (int)args.s1;
        a_hi = (int)args.s_end - 1;
    } else if (args.mode == BAND_PLAIN) {
        // a tile on anti-diagonal A holds the entry stages 64 A .. 64 A + 126
        const int64_t lo = (args.s1 - 2 * (BT - 1)) / BT;
        a_lo = (int)(lo > 0 ? lo : 0);
        const int64_t hi = (args.s_end - 1) / BT;
        a_hi = (int)(hi < a_hi ? hi : a_hi);
    }
    if (a_hi < a_lo) return G2D_OK;
    const int max_len = nTI < nTJ ? nTI : nTJ;
    dim3 grid((unsigned)max_len, (unsigned)(a_hi - a_lo + 1), (unsigned)(args.batch < 65535 ? args.batch : 65535));
    switch (args.mode) {
    case BAND_TILE: band_update_kernel<F, BAND_TILE><<<grid, BTH, 0, stream>>>(args, nTI, nTJ, a_lo); break;
    case BAND_PLAIN: band_update_kernel<F, BAND_PLAIN><<<grid, BTH, 0, stream>>>(args, nTI, nTJ, a_lo); break;
    default: band_update_kernel<F, BAND_GENERAL><<<grid, BTH, 0, stream>>>(args, nTI, nTJ, a_lo); break;
    }
    return check_launch();
}

template int launch_band_update<float>(const BandArgs<float> &, cudaStream_t);
template int launch_band_update<double>(const BandArgs<double> &, cudaStream_t);

}  // namespace g2d
