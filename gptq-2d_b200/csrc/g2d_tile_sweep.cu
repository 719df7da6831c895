// Fused tile sweep: one CTA rounds one TILE x TILE tile of the matrix, with the quantizer inside.
//
// Replaces, for the quantizers this library knows, the per-stage quantizer call and
// _push_kernel of the reference (gptq_2d.py:243-346, driven from :1342-1374).  Any order that
// respects "above and to the left first" gives the reference's result in exact arithmetic
// (gptq_2d_reference.py:166-200 prove it for two other orders), so the sweep is organised for
// the hardware instead of by global anti-diagonals:
//
//   * the host launches one grid per tile anti-diagonal; the tiles of one anti-diagonal are
//     independent, all feedback from earlier tiles is already in Y (right) and C (down);
//   * inside the CTA the tile lives in shared memory; warp a sweeps sub-tile (a, w - a) of the
//     sub-tile anti-diagonal w in registers, then all warps apply the finished sub-tiles'
//     feedback to the rest of the tile as small dense products;
//   * inside a sub-tile the 16 + 16 lanes of a warp own its columns and rows.  Lane j < 16 holds
//     the down feedback ("C") of column j, lane 16 + i the right feedback ("Y") of row i, both
//     skewed so that the entries of anti-diagonal s sit in register s mod 16 of every lane: the
//     stage loop is fully unrolled and indexes registers statically.
#include "g2d_common.cuh"

namespace g2d {

template <typename F>
__device__ __forceinline__ void mm16(F *__restrict__ D, const F *__restrict__ A, const F *__restrict__ B, int lane) {
    // D[16x16] += A[16x16] * B[16x16], all in shared memory with row stride LD; 2 x 4 outputs per lane.
    const int r = (lane >> 2) * 2, c = (lane & 3) * 4;
    F d[2][4];
#pragma unroll
    for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) d[x][y] = D[(r + x) * LD + c + y];
#pragma unroll
    for (int k = 0; k < SUB; ++k) {
        const F a0 = A[r * LD + k], a1 = A[(r + 1) * LD + k];
        F b[4];
#pragma unroll
        for (int y = 0; y < 4; ++y) b[y] = B[k * LD + c + y];
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            d[0][y] += a0 * b[y];
            d[1][y] += a1 * b[y];
        }
    }
#pragma unroll
    for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) D[(r + x) * LD + c + y] = d[x][y];
}

template <typename F>
__global__ void __launch_bounds__(NSUB * 32) tile_sweep_kernel(SweepArgs<F> P, int S) {
    extern __shared__ __align__(16) unsigned char g2d_smem[];
    F *Ys = reinterpret_cast<F *>(g2d_smem);  // X + right feedback; the errors E once a sub-tile is swept
    F *Cs = Ys + TILE * LD;                   // down feedback; the completed C once a sub-tile is swept
    F *LUs = Cs + TILE * LD;                  // strict lower part: L[I, I]; strict upper part: U[J, J]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = lane & 15, half = lane >> 4;
    const int I = max(0, S - P.nJ + 1) + (int)blockIdx.x, J = S - I;
    const int64_t i0 = (int64_t)I * TILE, j0 = (int64_t)J * TILE;
    const int64_t m = P.m, n = P.n;

    for (int64_t batch = blockIdx.y; batch < P.batch; batch += gridDim.y) {
        F *yg = P.y + batch * m * n, *cg = P.c + batch * m * n, *eg = P.e + batch * m * n;
        const F *lg = P.l + (P.l_off ? P.l_off[batch] : 0);
        const F *ug = P.u + (P.u_off ? P.u_off[batch] : 0);
        const F *sg = P.kind == G2D_Q_AFFINE ? P.scale + (P.scale_off ? P.scale_off[batch] : 0) : nullptr;
        const F *zg = P.kind == G2D_Q_AFFINE ? P.zero + (P.zero_off ? P.zero_off[batch] : 0) : nullptr;
        const F *fg = P.kind == G2D_Q_FORCED ? P.forced + batch * m * n : nullptr;
        F *pre = P.y_pre ? P.y_pre + batch * m * n : nullptr;

        // ---- load the tile: consecutive threads read consecutive columns ----
        for (int idx = tid; idx < TILE * TILE; idx += NSUB * 32) {
            const int r = idx / TILE, c = idx % TILE;
            const int64_t gi = i0 + r, gj = j0 + c;
            const bool in = gi < m && gj < n;
            Ys[r * LD + c] = in ? yg[gi * n + gj] : (F)0;
            Cs[r * LD + c] = in ? cg[gi * n + gj] : (F)0;
            F coef = (F)0;
            if (r > c) {
                if (gi < m) coef = lg[gi * m + i0 + c];
            } else if (r < c) {
                if (gj < n) coef = ug[(j0 + r) * n + gj];
            }
            LUs[r * LD + c] = coef;
        }
        __syncthreads();

        F sc[SUB], zp[SUB];  // quantizer parameters of this lane's entries, skewed like acc
        bool have_params = false;

        for (int w = 0; w < 2 * NSUB - 1; ++w) {
            const int a = warp, b = w - warp;
            if (b >= 0 && b < NSUB) {
                const int r0 = a * SUB, c0 = b * SUB;
                if (!have_params && P.kind != G2D_Q_ROUND) {
#pragma unroll
                    for (int r = 0; r < SUB; ++r) {
                        const int o = (r - k) & (SUB - 1);
                        const int64_t gi = i0 + r0 + (half ? k : o), gj = j0 + c0 + (half ? o : k);
                        const bool in = gi < m && gj < n;
                        if (P.kind == G2D_Q_AFFINE) {
                            sc[r] = in ? sg[gi * P.srs + gj * P.scs] : (F)1;
                            zp[r] = in ? zg[gi * P.zrs + gj * P.zcs] : (F)0;
                        } else {
                            sc[r] = in ? fg[gi * n + gj] : (F)0;
                        }
                    }
                }
                F acc[SUB];
#pragma unroll
                for (int r = 0; r < SUB; ++r) {
                    const int o = (r - k) & (SUB - 1);
                    acc[r] = half ? Ys[(r0 + k) * LD + c0 + o] : Cs[(r0 + o) * LD + c0 + k];
                }
                const int base = half ? c0 : r0, step = half ? 1 : LD;
#pragma unroll
                for (int s = 0; s < 2 * SUB - 1; ++s) {
                    const int r = s & (SUB - 1);
                    const int src = s - k;
                    const bool active = src >= 0 && src < SUB;
                    const int srcw = src & (SUB - 1);
                    // column owner j = k needs the Y accumulator of row src; row owner i = k the C accumulator of column src
                    const F other = __shfl_sync(0xffffffffu, acc[r], half ? srcw : SUB + srcw);
                    const F yacc = half ? acc[r] : other, cacc = half ? other : acc[r];
                    const F yv = yacc + cacc;
                    const int li = half ? k : srcw, lj = half ? srcw : k;
                    const int64_t gi = i0 + r0 + li, gj = j0 + c0 + lj;
                    const bool in = active && gi < m && gj < n;
                    F z;
                    if (P.kind == G2D_Q_AFFINE) z = affine_value(yv, sc[r], zp[r], P.qmin, P.qmax);
                    else if (P.kind == G2D_Q_FORCED) z = sc[r];
                    else z = rint_even(yv);
                    const F ev = in ? z - yv : (F)0;
                    const F cc = cacc + ev;
                    if (active) {
                        if (half) {
                            Cs[(r0 + li) * LD + c0 + lj] = cc;
                            if (in) {
                                yg[gi * n + gj] = z;
                                if (pre) pre[gi * n + gj] = yv;
                            }
                        } else {
                            Ys[(r0 + li) * LD + c0 + lj] = ev;
                        }
                    }
                    // push: the column owner sends its error down through L, the row owner its completed C right through U
                    const F val = half ? cc : ev;
                    const F *cp = LUs + (base + srcw) * LD + base + srcw;
                    constexpr int kMaxPush = SUB - 1;
                    const int dd_hi = s < SUB ? kMaxPush : 2 * SUB - 2 - s;  // static bound: src >= s - (SUB - 1)
#pragma unroll
                    for (int dd = 1; dd <= kMaxPush; ++dd) {
                        if (dd <= dd_hi) {
                            if (active && dd <= SUB - 1 - src) acc[(r + dd) & (SUB - 1)] += cp[dd * step] * val;
                        }
                    }
                }
            }
            // fetch the parameters of the next sub-tile of this warp while the updates run
            {
                const int bn = w + 1 - warp;
                have_params = false;
                if (bn >= 0 && bn < NSUB && P.kind != G2D_Q_ROUND) {
                    const int r0 = warp * SUB, c0 = bn * SUB;
#pragma unroll
                    for (int r = 0; r < SUB; ++r) {
                        const int o = (r - k) & (SUB - 1);
                        const int64_t gi = i0 + r0 + (half ? k : o), gj = j0 + c0 + (half ? o : k);
                        const bool in = gi < m && gj < n;
                        if (P.kind == G2D_Q_AFFINE) {
                            sc[r] = in ? sg[gi * P.srs + gj * P.scs] : (F)1;
                            zp[r] = in ? zg[gi * P.zrs + gj * P.zcs] : (F)0;
                        } else {
                            sc[r] = in ? fg[gi * n + gj] : (F)0;
                        }
                    }
                    have_params = true;
                }
            }
            __syncthreads();
            // ---- apply the finished sub-tiles to the rest of the tile ----
            if (w < 2 * NSUB - 2) {
                int count = 0;
                for (int ap = 0; ap < NSUB; ++ap) {
                    for (int bp = 0; bp < NSUB; ++bp) {
                        if (ap + bp <= w) continue;
                        const int as = w - bp, bs = w - ap;
                        const bool down = as >= 0 && as < NSUB, right = bs >= 0 && bs < NSUB;
                        if (!down && !right) continue;
                        if ((count++ & (NSUB - 1)) != warp) continue;
                        if (down)  // C[ap, bp] += L[ap, as] E[as, bp]
                            mm16(Cs + ap * SUB * LD + bp * SUB, LUs + ap * SUB * LD + as * SUB, Ys + as * SUB * LD + bp * SUB, lane);
                        if (right)  // Y[ap, bp] += C[ap, bs] U[bs, bp]
                            mm16(Ys + ap * SUB * LD + bp * SUB, Cs + ap * SUB * LD + bs * SUB, LUs + bs * SUB * LD + bp * SUB, lane);
                    }
                }
                __syncthreads();
            }
        }

        // ---- store the errors and the completed C of the tile; Z went out entry by entry ----
        for (int idx = tid; idx < TILE * TILE; idx += NSUB * 32) {
            const int r = idx / TILE, c = idx % TILE;
            const int64_t gi = i0 + r, gj = j0 + c;
            if (gi < m && gj < n) {
                eg[gi * n + gj] = Ys[r * LD + c];
                cg[gi * n + gj] = Cs[r * LD + c];
            }
        }
        __syncthreads();
    }
}

template <typename F>
int launch_tile_sweep(const SweepArgs<F> &args, int S, cudaStream_t stream) {
    // the opt-in to more than 48 KB of dynamic shared memory is per device
    static bool configured[64] = {};
    const size_t smem = sizeof(F) * 3 * TILE * LD;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return G2D_ERR_CUDA;
    if (!configured[device]) {
        if (cudaFuncSetAttribute(tile_sweep_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return G2D_ERR_CUDA;
        configured[device] = true;
    }
    const int i_lo = S - args.nJ + 1 > 0 ? S - args.nJ + 1 : 0;
    const int i_hi = S + 1 < args.nI ? S + 1 : args.nI;
    dim3 grid((unsigned)(i_hi - i_lo), (unsigned)(args.batch < 65535 ? args.batch : 65535));
    tile_sweep_kernel<F><<<grid, NSUB * 32, smem, stream>>>(args, S);
    return check_launch();
}

template int launch_tile_sweep<float>(const SweepArgs<float> &, int, cudaStream_t);
template int launch_tile_sweep<double>(const SweepArgs<double> &, int, cudaStream_t);

}  // namespace g2d
