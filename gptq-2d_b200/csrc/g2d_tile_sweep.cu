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
//   * inside the CTA the tile lives in shared memory; the 16 x 16 sub-tiles are taken on a sub-tile wavefront: the
//     up to four sub-tiles of one sub-tile anti-diagonal are swept in registers by the four half-warps of warps 0 and 1.
//     These two warps are the critical path of the whole sweep and do nothing but the rounding stages: four helper
//     warps, one per sub-tile row, carry everything else while a sub-tile anti-diagonal is swept (the quantizer
//     parameters of the next one, the feedback of finished sub-tiles into sub-tiles two or more anti-diagonals ahead,
//     the feedback of the neighbour tiles) and, between two sweeps, the one product pair per sub-tile that cannot
//     be formed earlier: the feedback of the anti-diagonal just swept into the next one;
//   * inside a sub-tile lane k of the half-warp owns column k (the down feedback, "C") and row k (the right feedback,
//     "Y"), both skewed so that the entries of anti-diagonal s sit in register s mod 16 of every lane: the stage loop
//     runs in groups of ROLL stages that index registers statically, and the registers are renamed by moving them
//     after every group; two shuffles per stage exchange the row accumulator and the completed C with the partner
//     lane.  The feedback coefficients of a sub-tile come from zero-padded copies of the diagonal blocks of L and
//     U^T, so the pushes need no bounds predicates: out-of-range pushes multiply by zero;
//   * pipelined schedule: a tile also adds the far-feedback planes as it loads, and the feedback between neighbour
//     tiles of consecutive tile anti-diagonals travels as a push: the helper warps of tile (I, J) form, from the
//     errors and the completed C in shared memory,  L[I + 1, I] E[I, J]  and  C[I, J] U[J, J + 1]  while the tile is
//     still being swept and store them into two planes of their own, which the tiles (I + 1, J) and (I, J + 1) add
//     as they load one launch later.  No load from another tile's results sits on a tile's critical path.
#include <type_traits>

#include "g2d_common.cuh"

namespace g2d {

// Push coefficients of a 16 x 16 diagonal block, one row per source p: entry [p][dd] is the coefficient that carries
// the value of source p to the receiver dd places further (L[p + dd][p] or U[p][p + dd]), zero for dd = 0 and past the
// block's end.  A lane fetches its row with four 16-byte loads; a row stride of 20 keeps eight lanes on distinct banks.
constexpr int DLD = SUB + 4;            // row stride
constexpr int DBLK = SUB * DLD;         // elements per block
constexpr int ROLL = 4;                 // rounding stages per iteration of the stage loop
constexpr int SWEEPERS = NSUB / 2;      // warps that sweep: one half-warp per sub-tile row
constexpr int HELPERS = NSUB;           // warps that feed them: one per sub-tile row
constexpr int TTH = (SWEEPERS + HELPERS) * 32;  // threads per CTA
constexpr int LANES = SWEEPERS * 32;    // sweeping lanes
constexpr int ZLD = SUB;                // row stride of the staging blocks of the rounded values (the walk down an anti-diagonal moves 15 words: no conflicts)

template <typename F>
__device__ __forceinline__ void load4(const F *p, F (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float *p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<double>(const double *p, double (&v)[4]) {
    const double2 a = *reinterpret_cast<const double2 *>(p), b = *reinterpret_cast<const double2 *>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename F>
__device__ __forceinline__ void store4(F *p, const F (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<double>(double *p, const double (&v)[4]) {
    *reinterpret_cast<double2 *>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2 *>(p + 2) = make_double2(v[2], v[3]);
}

template <typename F>
__device__ __forceinline__ void mm16(F *__restrict__ D, const F *__restrict__ A, const F *__restrict__ B, int lane) {
    // D[16x16] += A[16x16] * B[16x16], all in shared memory with row stride LD; one warp, 2 x 4 outputs per lane
    const int r = (lane >> 2) * 2, c = (lane & 3) * 4;
    F d0[4], d1[4];
    load4(D + r * LD + c, d0);
    load4(D + (r + 1) * LD + c, d1);
#pragma unroll
    for (int k = 0; k < SUB; k += 4) {
        F a0[4], a1[4];
        load4(A + r * LD + k, a0);
        load4(A + (r + 1) * LD + k, a1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            F b[4];
            load4(B + (k + kk) * LD + c, b);
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                d0[y] += a0[kk] * b[y];
                d1[y] += a1[kk] * b[y];
            }
        }
    }
    store4(D + r * LD + c, d0);
    store4(D + (r + 1) * LD + c, d1);
}

// The one or two products that carry finished sub-tiles into sub-tile (ap, bp): the errors of (as, bp) down through
// L[ap, as] into C, then the completed C of (ap, bs) right through U[bs, bp] into Y; a source index outside 0 .. NSUB - 1
// means there is no such source.  One warp; a loop, so that the product's code exists once per call site.
template <typename F>
__device__ __forceinline__ void carry_into(F *Ys, F *Cs, const F *LUs, int ap, int bp, int as, int bs, int lane) {
#pragma unroll 1
    for (int prod = 0; prod < 2; ++prod) {
        const int src = prod == 0 ? as : bs;
        if (src < 0 || src >= NSUB) continue;
        F *D = (prod == 0 ? Cs : Ys) + ap * SUB * LD + bp * SUB;
        const F *A = prod == 0 ? LUs + ap * SUB * LD + src * SUB : Cs + ap * SUB * LD + src * SUB;
        const F *B = prod == 0 ? Ys + src * SUB * LD + bp * SUB : LUs + src * SUB * LD + bp * SUB;
        mm16(D, A, B, lane);
    }
}

// The products of the neighbour push: the 2 x 4 outputs of a lane stay in registers.  d += A B with A and B in shared
// memory (row stride LD), and the same with the lane's two rows of A held in registers.
template <typename F>
__device__ __forceinline__ void mm16_acc(F (&d0)[4], F (&d1)[4], const F *__restrict__ A, const F *__restrict__ B, int lane) {
    const int r = (lane >> 2) * 2, c = (lane & 3) * 4;
#pragma unroll
    for (int k = 0; k < SUB; k += 4) {
        F a0[4], a1[4];
        load4(A + r * LD + k, a0);
        load4(A + (r + 1) * LD + k, a1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            F b[4];
            load4(B + (k + kk) * LD + c, b);
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                d0[y] += a0[kk] * b[y];
                d1[y] += a1[kk] * b[y];
            }
        }
    }
}
template <typename F>
__device__ __forceinline__ void mm16_areg(F (&d0)[4], F (&d1)[4], const F *a0, const F *a1, const F *__restrict__ B, int lane) {
    // a0 / a1: this lane's quarter of its two rows of A (columns 4 (lane % 4) .. + 3); the four lanes that share the
    // rows hand each other their quarters by shuffle
    const int c = (lane & 3) * 4;
#pragma unroll
    for (int k = 0; k < SUB; ++k) {
        F b[4];
        load4(B + k * LD + c, b);
        const F v0 = __shfl_sync(0xffffffffu, a0[k & 3], k >> 2, 4), v1 = __shfl_sync(0xffffffffu, a1[k & 3], k >> 2, 4);
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            d0[y] += v0 * b[y];
            d1[y] += v1 * b[y];
        }
    }
}
// Stores a lane's 2 x 4 outputs of a 16 x 16 block at `dst` (row stride ld); rows / columns from rows_left / cols_left on lie
// outside the matrix.  `vec`: rows are 16-byte aligned and columns come in whole groups of four.
template <typename F>
__device__ __forceinline__ void store_block(F *dst, int64_t ld, const F (&d0)[4], const F (&d1)[4], int lane, int64_t rows_left, int64_t cols_left, bool vec) {
    const int r = (lane >> 2) * 2, c = (lane & 3) * 4;
    if (vec) {
        if (c < cols_left) {
            if (r < rows_left) store4(dst + r * ld + c, d0);
            if (r + 1 < rows_left) store4(dst + (r + 1) * ld + c, d1);
        }
    } else {
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            if (c + y < cols_left) {
                if (r < rows_left) dst[r * ld + c + y] = d0[y];
                if (r + 1 < rows_left) dst[(r + 1) * ld + c + y] = d1[y];
            }
        }
    }
}

template <typename F, int KIND>
__global__ void __launch_bounds__(TTH) tile_sweep_kernel(SweepArgs<F> P, int S, int i_first, int i_step) {
    extern __shared__ __align__(16) unsigned char g2d_smem[];
    F *Ys = reinterpret_cast<F *>(g2d_smem);  // X + right feedback; the errors E once a sub-tile is swept
    F *Cs = Ys + TILE * LD;                   // down feedback; the completed C once a sub-tile is swept
    F *LUs = Cs + TILE * LD;                  // strict lower part: L[I, I]; strict upper part: U[J, J]
    F *Dg = LUs + TILE * LD;                  // [2][NSUB] zero-padded diagonal blocks: L[a, a] and U[b, b]^T, strictly lower
    F *Ubs = Dg + 2 * NSUB * DBLK;            // pipelined schedule: U[J, J + 1], the right neighbour's coupling block
    F *Ps = Ubs + TILE * LD;                   // [3][SUB][LANES]: quantizer parameters of the sweeping lanes, by register number
    F *Zst = Ps + 3 * SUB * LANES;            // [NSUB][SUB][ZLD]: rounded values of the sub-tiles being swept, written out by the helpers after the sweep
    unsigned *Pv = reinterpret_cast<unsigned *>(Zst + NSUB * SUB * ZLD);  // [2][LANES] registers holding entries inside the matrix, one word per half of the registers; [2][SWEEPERS] reciprocal division allowed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = lane & 15, half = lane >> 4;
    const int I = i_first + i_step * (int)blockIdx.x, J = S - I;  // tiles of the anti-diagonal S, every one or every second
    const int64_t i0 = (int64_t)I * TILE, j0 = (int64_t)J * TILE;
    const int64_t m = P.m, n = P.n;
    const bool full = i0 + TILE <= m && j0 + TILE <= n;
    const bool sweeper = warp < SWEEPERS;
    const int helper = warp - SWEEPERS;  // 0 .. HELPERS - 1 for the helper warps: the sub-tile row the warp feeds

    for (int64_t batch = blockIdx.y; batch < P.batch; batch += gridDim.y) {
        F *yg = P.y + batch * m * n, *cg = P.c + batch * m * n, *eg = P.e + batch * m * n;
        const F *lg = P.l + (P.l_off ? P.l_off[batch] : 0);
        const F *ug = P.u + (P.u_off ? P.u_off[batch] : 0);
        const F *sg = KIND == G2D_Q_AFFINE ? P.scale + (P.scale_off ? P.scale_off[batch] : 0) : nullptr;
        const F *zg = KIND == G2D_Q_AFFINE ? P.zero + (P.zero_off ? P.zero_off[batch] : 0) : nullptr;
        const F *fg = KIND == G2D_Q_FORCED ? P.forced + batch * m * n : nullptr;
        F *pre = P.y_pre ? P.y_pre + batch * m * n : nullptr;
        const F *yfg = P.yf ? P.yf + batch * m * n : nullptr, *cfg = P.yf ? P.cf + batch * m * n : nullptr;
        // neighbour push (pipelined schedule): what this tile receives and what it owes
        F *yng = P.yn ? P.yn + batch * m * n : nullptr, *cng = P.yn ? P.cn + batch * m * n : nullptr;
        const bool gets_right = yng != nullptr && J > 0, gets_down = yng != nullptr && I > 0;
        const bool owes_right = yng != nullptr && J + 1 < P.nJ, owes_down = yng != nullptr && I + 1 < P.nI;

        // ---- quantizer parameters, prepared by the helper warps ----
        // Helper warp h prepares, for the sweeping lane of its own lane number in sweeping warp h mod SWEEPERS, half
        // h / SWEEPERS of that lane's registers: register r holds entry ((r - k) mod 16, k) of the lane's sub-tile.
        // Scale, zero point and, for the float affine quantizer, the refined reciprocal of the scale (see
        // affine_value_rcp) wait in shared memory by register number, with the bits that say which registers hold
        // entries inside the matrix and the warp-wide decision whether every scale is in the range where the reciprocal
        // form of the division is safe.  The loads are issued one sub-tile anti-diagonal ahead and travel while the
        // helper does its other work.
        constexpr int PR = SUB / (HELPERS / SWEEPERS);  // registers per helper lane
        F sc[PR], zp[PR], rc[PR];
        bool pfast = true;
        unsigned pvalid = 0;
        const int p_warp = helper & (SWEEPERS - 1), p_part = helper / SWEEPERS;  // helpers only
        const int p_lane = p_warp * 32 + lane;
        const int p_a = 2 * p_warp + half;  // sub-tile row of the lane prepared for
        auto fetch_params = [&](int w_next) {
            const int b_raw = w_next - p_a;
            const int b = b_raw >= 0 && b_raw < NSUB ? b_raw : 0;  // a half-warp without a sub-tile gets valid dummies and stays masked
            const int r0 = p_a * SUB, c0 = b * SUB;
            unsigned bits = 0;
#pragma unroll
            for (int x = 0; x < PR; ++x) {
                const int r = p_part * PR + x, o = (r - k) & (SUB - 1);
                const int64_t gi = i0 + r0 + o, gj = j0 + c0 + k;
                const bool in = full || (gi < m && gj < n);
                bits |= in ? (1u << r) : 0u;
                // entries outside the matrix load a value from inside it (no select waits on the load here) and get
                // their neutral parameters in finish_params
                const int64_t ci = gi < m ? gi : m - 1, cj = gj < n ? gj : n - 1;
                if (KIND == G2D_Q_AFFINE) {
                    sc[x] = sg[ci * P.srs + cj * P.scs];
                    zp[x] = zg[ci * P.zrs + cj * P.zcs];
                } else if (KIND == G2D_Q_FORCED) {
                    sc[x] = fg[ci * n + cj];
                }
            }
            pvalid = bits;
        };
        auto finish_params = [&]() {
#pragma unroll
            for (int x = 0; x < PR; ++x) {
                const bool in = (pvalid >> (p_part * PR + x)) & 1u;
                if (KIND == G2D_Q_AFFINE) {
                    sc[x] = in ? sc[x] : (F)1;
                    zp[x] = in ? zp[x] : (F)0;
                } else if (KIND == G2D_Q_FORCED) {
                    sc[x] = in ? sc[x] : (F)0;
                }
            }
            if (KIND == G2D_Q_AFFINE && sizeof(F) == sizeof(float)) {
                bool normal = true;
#pragma unroll
                for (int x = 0; x < PR; ++x) {
                    const float sv = (float)sc[x], av = fabsf(sv);
                    normal = normal && av > 1e-18f && av < 1e18f;
                    float v = __frcp_rn(sv);
                    v = fmaf(fmaf(-sv, v, 1.f), v, v);  // one Newton step: the reciprocal to within half an ulp
                    rc[x] = (F)v;
                }
                pfast = __all_sync(0xffffffffu, normal);
            }
        };
        auto store_params = [&]() {
#pragma unroll
            for (int x = 0; x < PR; ++x) {
                const int r = p_part * PR + x;
                if (KIND != G2D_Q_ROUND) Ps[(0 * SUB + r) * LANES + p_lane] = sc[x];
                if (KIND == G2D_Q_AFFINE) {
                    Ps[(1 * SUB + r) * LANES + p_lane] = zp[x];
                    Ps[(2 * SUB + r) * LANES + p_lane] = rc[x];
                }
            }
            Pv[p_part * LANES + p_lane] = pvalid;
            if (lane == 0) Pv[2 * LANES + p_part * SWEEPERS + p_warp] = pfast ? 1u : 0u;
        };
        if (!sweeper) fetch_params(0);

        constexpr bool PUSH = sizeof(F) == sizeof(float);  // the neighbour push exists for float (pipelined schedule) only

        // ---- load the tile; all global loads of a pass are issued before its shared-memory stores ----
        const bool vec = full && (n % 4 == 0) && (m % 4 == 0) &&
                         ((reinterpret_cast<uintptr_t>(yg) | reinterpret_cast<uintptr_t>(cg) | reinterpret_cast<uintptr_t>(eg) |
                           reinterpret_cast<uintptr_t>(lg) | reinterpret_cast<uintptr_t>(ug)) % (4 * sizeof(F)) == 0);
        if (vec) {
            constexpr int VECS = TILE * TILE / 4;              // vectors per array
            constexpr int PER = (VECS + TTH - 1) / TTH;        // per thread, the last one partly
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                F va[PER][4], vb[PER][4];
#pragma unroll
                for (int t = 0; t < PER; ++t) {
                    const int idx = t * TTH + tid, r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                    if (idx >= VECS) continue;
                    if (pass == 0) {
                        load4(yg + (i0 + r) * n + j0 + c, va[t]);
                        load4(cg + (i0 + r) * n + j0 + c, vb[t]);
                    } else {
                        load4(lg + (i0 + r) * m + i0 + c, va[t]);
                        load4(ug + (j0 + r) * n + j0 + c, vb[t]);
                    }
                }
                if (pass == 0 && yfg != nullptr) {
                    // the far planes and what the left and the upper neighbour pushed one launch ago: all loads are
                    // issued before the first addition, so that the tile waits for global memory once
                    F fa[PER][4], fb[PER][4], na[PER][4], nb[PER][4];
#pragma unroll
                    for (int t = 0; t < PER; ++t) {
                        const int idx = t * TTH + tid, r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                        if (idx >= VECS) continue;
                        load4(yfg + (i0 + r) * n + j0 + c, fa[t]);
                        load4(cfg + (i0 + r) * n + j0 + c, fb[t]);
                        if constexpr (PUSH) {
#pragma unroll
                            for (int x = 0; x < 4; ++x) na[t][x] = nb[t][x] = (F)0;
                            if (gets_right) load4(yng + (i0 + r) * n + j0 + c, na[t]);
                            if (gets_down) load4(cng + (i0 + r) * n + j0 + c, nb[t]);
                        }
                    }
#pragma unroll
                    for (int t = 0; t < PER; ++t) {
                        if (t * TTH + tid >= VECS) continue;
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            va[t][x] += fa[t][x];
                            vb[t][x] += fb[t][x];
                            if constexpr (PUSH) {
                                va[t][x] += na[t][x];
                                vb[t][x] += nb[t][x];
                            }
                        }
                    }
                }
                if (pass == 1 && owes_right) {
#pragma unroll
                    for (int t = 0; t < PER; ++t) {
                        const int idx = t * TTH + tid, r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                        if (idx >= VECS) continue;
                        F uv[4] = {(F)0, (F)0, (F)0, (F)0};
                        if (j0 + TILE + c < n) load4(ug + (j0 + r) * n + j0 + TILE + c, uv);
                        store4(Ubs + r * LD + c, uv);
                    }
                }
#pragma unroll
                for (int t = 0; t < PER; ++t) {
                    const int idx = t * TTH + tid, r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                    if (idx >= VECS) continue;
                    if (pass == 0) {
                        store4(Ys + r * LD + c, va[t]);
                        store4(Cs + r * LD + c, vb[t]);
                    } else {
                        F lu[4];
#pragma unroll
                        for (int x = 0; x < 4; ++x) lu[x] = r > c + x ? va[t][x] : (r < c + x ? vb[t][x] : (F)0);
                        store4(LUs + r * LD + c, lu);
                    }
                }
            }
        } else {
            constexpr int UN = 8;
            for (int base = 0; base < TILE * TILE; base += TTH * UN) {
                F vy[UN], vc[UN], vl[UN];
#pragma unroll
                for (int t = 0; t < UN; ++t) {
                    const int idx = base + t * TTH + tid, r = idx / TILE, c = idx % TILE;
                    const int64_t gi = i0 + r, gj = j0 + c;
                    const bool in = idx < TILE * TILE && gi < m && gj < n;
                    vy[t] = in ? yg[gi * n + gj] : (F)0;
                    vc[t] = in ? cg[gi * n + gj] : (F)0;
                    if (in && yfg != nullptr) {
                        vy[t] += yfg[gi * n + gj];
                        vc[t] += cfg[gi * n + gj];
                        if (gets_right) vy[t] += yng[gi * n + gj];
                        if (gets_down) vc[t] += cng[gi * n + gj];
                    }
                    vl[t] = (F)0;
                    if (idx < TILE * TILE) {
                        if (r > c) {
                            if (gi < m) vl[t] = lg[gi * m + i0 + c];
                        } else if (r < c) {
                            if (gj < n) vl[t] = ug[(j0 + r) * n + gj];
                        }
                    }
                }
#pragma unroll
                for (int t = 0; t < UN; ++t) {
                    const int idx = base + t * TTH + tid, r = idx / TILE, c = idx % TILE;
                    if (idx >= TILE * TILE) continue;
                    Ys[r * LD + c] = vy[t];
                    Cs[r * LD + c] = vc[t];
                    LUs[r * LD + c] = vl[t];
                }
            }
            if (owes_right)
                for (int idx = tid; idx < TILE * TILE; idx += TTH) {
                    const int r = idx / TILE, c = idx % TILE;
                    Ubs[r * LD + c] = (j0 + r < n && j0 + TILE + c < n) ? ug[(j0 + r) * n + j0 + TILE + c] : (F)0;
                }
        }
        __syncthreads();
        for (int idx = tid; idx < 2 * NSUB * DBLK; idx += TTH) {
            const int which = idx / (NSUB * DBLK), blk = idx / DBLK % NSUB, p = idx % DBLK / DLD, dd = idx % DLD;
            F v = (F)0;
            if (dd >= 1 && dd < SUB && p + dd < SUB)
                v = which == 0 ? LUs[(blk * SUB + p + dd) * LD + blk * SUB + p] : LUs[(blk * SUB + p) * LD + blk * SUB + p + dd];
            Dg[idx] = v;
        }
        if (!sweeper) {
            finish_params();
            store_params();
        }
        __syncthreads();

        // Sweep of the sub-tiles.  A half-warp (16 lanes) sweeps one sub-tile, so warps 0 and 1 hold the up to four
        // sub-tiles of a sub-tile anti-diagonal: half-warp h of warp w2 takes sub-tile row a = 2 w2 + h.  Lane k owns
        // column k (down feedback, "C") and row k (right feedback, "Y") of its sub-tile, both skewed so that the entries of
        // anti-diagonal s sit in register s mod 16.  At stage s lane k rounds its column's entry (p, k), p = s - k; the
        // lane that owns row p is lane p, and lane p in turn rounds (k, p), the entry of this lane's row: the two lanes
        // exchange the row accumulator before rounding and the completed C after it.
        // The two roles run the same sequence of barriers from loops of their own, so that neither holds the other's registers.
        if (sweeper) {
            for (int w = 0; w < 2 * NSUB - 1; ++w) {
                const int sub_a = 2 * warp + half;
                const int b_raw = w - sub_a;
                const bool tile_ok = b_raw >= 0 && b_raw < NSUB;  // a half-warp without a sub-tile runs along with everything masked
                const int b = tile_ok ? b_raw : 0;
                const int r0 = sub_a * SUB, c0 = b * SUB;
                const unsigned valid_bits = Pv[tid] | Pv[LANES + tid];
                const bool fast_division = (Pv[2 * LANES + warp] & Pv[2 * LANES + SWEEPERS + warp]) != 0u;
                F cacc[SUB], yacc[SUB];
#pragma unroll
                for (int r = 0; r < SUB; ++r) {
                    const int o = (r - k) & (SUB - 1);
                    cacc[r] = Cs[(r0 + o) * LD + c0 + k];
                    yacc[r] = Ys[(r0 + k) * LD + c0 + o];
                }
                // entry (s - k, k) of the sub-tile: a lane-constant address plus s rows
                const int entry0 = (r0 - k) * LD + c0 + k;
                F *pre_ptr = pre ? pre + (i0 + r0 - k) * n + j0 + c0 + k : nullptr;
                const int zst0 = (r0 - k) * ZLD + k;
                const F *const dgl = Dg + sub_a * DBLK, *const dgu = Dg + (NSUB + b) * DBLK;
                // The 32 stages in groups of ROLL: inside a group the registers are indexed statically, after it they are
                // renamed by moving them ROLL places, so that the loop body is ROLL stages long (the fully unrolled form
                // is 25 KB of straight-line code per pass that no instruction cache level close to the scheduler holds).
                auto stages = [&](auto fast_tag) {
                    constexpr bool FASTDIV = decltype(fast_tag)::value;
#pragma unroll 1
                    for (int group = 0; group < 2 * SUB / ROLL; ++group) {
                        const int s_first = group * ROLL;
#pragma unroll
                        for (int j = 0; j < ROLL; ++j) {
                            const int s = s_first + j, r = s & (SUB - 1);
                            const int p = s - k;  // row of this lane's column entry = column of its row entry = partner lane
                            const bool active = tile_ok && p >= 0 && p < SUB;
                            const int pw = p & (SUB - 1);
                            const F yrow = __shfl_sync(0xffffffffu, yacc[j], pw, SUB);  // Y accumulator of (p, k) from the owner of row p
                            const F yv = yrow + cacc[j];
                            const bool ok = active && ((valid_bits >> r) & 1u);
                            F z;
                            if (KIND == G2D_Q_AFFINE) {
                                const F scv = Ps[(0 * SUB + r) * LANES + tid], zpv = Ps[(1 * SUB + r) * LANES + tid];
                                z = FASTDIV ? affine_value_rcp(yv, scv, zpv, Ps[(2 * SUB + r) * LANES + tid], P.qmin, P.qmax) : affine_value(yv, scv, zpv, P.qmin, P.qmax);
                            } else if (KIND == G2D_Q_FORCED) {
                                z = Ps[(0 * SUB + r) * LANES + tid];
                            } else {
                                z = rint_even(yv);
                            }
                            const F ev = ok ? z - yv : (F)0;
                            const F cc = cacc[j] + ev;
                            const F ccrow = __shfl_sync(0xffffffffu, cc, pw, SUB);  // completed C of (k, p), rounded by lane p
                            if (active) {
                                Ys[entry0 + s * LD] = ev;
                                Cs[entry0 + s * LD] = cc;
                                Zst[zst0 + s * ZLD] = z;
                            }
                            if (ok && pre_ptr) pre_ptr[(int64_t)s * n] = yv;
                            // pushes: the error down column k through L, the completed C of (k, p) right along row k through U;
                            // rows past the block's end read the zero padding, inactive lanes push zero
                            const F vcol = active ? ev : (F)0, vrow = active ? ccrow : (F)0;
                            F kl[SUB], ku[SUB];
#pragma unroll
                            for (int v4 = 0; v4 < SUB; v4 += 4) {
                                F t[4];
                                load4(dgl + pw * DLD + v4, t);
#pragma unroll
                                for (int x = 0; x < 4; ++x) kl[v4 + x] = t[x];
                                load4(dgu + pw * DLD + v4, t);
#pragma unroll
                                for (int x = 0; x < 4; ++x) ku[v4 + x] = t[x];
                            }
#pragma unroll
                            for (int dd = 1; dd < SUB; ++dd) {
                                cacc[(j + dd) & (SUB - 1)] += kl[dd] * vcol;
                                yacc[(j + dd) & (SUB - 1)] += ku[dd] * vrow;
                            }
                        }
                        // rename: what was register i + ROLL is register i from here on
                        F keep_c[ROLL], keep_y[ROLL];
#pragma unroll
                        for (int i = 0; i < ROLL; ++i) { keep_c[i] = cacc[i]; keep_y[i] = yacc[i]; }
#pragma unroll
                        for (int i = 0; i < SUB - ROLL; ++i) { cacc[i] = cacc[i + ROLL]; yacc[i] = yacc[i + ROLL]; }
#pragma unroll
                        for (int i = 0; i < ROLL; ++i) { cacc[SUB - ROLL + i] = keep_c[i]; yacc[SUB - ROLL + i] = keep_y[i]; }
                    }
                };
                if (fast_division) stages(std::true_type{});
                else stages(std::false_type{});
                __syncthreads();
                if (w + 1 < 2 * NSUB - 1) __syncthreads();  // the helpers carry the anti-diagonal just swept into the next one
            }
        } else {
            // ---- neighbour push: registers of the helper warps (float, pipelined schedule) ----
            // Helper warp h keeps, in the layout of mm16 (rows 2 (lane / 4) and the next one), its two rows of the strip
            // L[I + 1, I](rows 16 h ..) for the down push (of each block of 16 columns the four that belong to lane % 4:
            // the four lanes of a row pair share them by shuffle), the running sums of the right push of sub-tile row h (four blocks;
            // not for the last row, whose four blocks are spread over the four helpers so that the work left after the
            // last sweep is one product each), and the last column's down push up to its last term.
            F lb0[PUSH ? TILE / 4 : 1], lb1[PUSH ? TILE / 4 : 1];
            F yn0[PUSH ? NSUB : 1][4], yn1[PUSH ? NSUB : 1][4], y30[4], y31[4], c30[4], c31[4];
            if constexpr (PUSH) {
#pragma unroll
                for (int y = 0; y < 4; ++y) {
#pragma unroll
                    for (int cb = 0; cb < NSUB; ++cb) yn0[cb][y] = yn1[cb][y] = (F)0;
                    y30[y] = y31[y] = c30[y] = c31[y] = (F)0;
                }
            }
            for (int w = 0; w < 2 * NSUB - 1; ++w) {
                const bool more = w + 1 < 2 * NSUB - 1;
                // Helper warp of sub-tile row ap, while sub-tile anti-diagonal w is swept.  Everything written here goes
                // to sub-tiles of row ap on later anti-diagonals, which no other warp touches before the barrier.
                const int ap = helper;
                if (more) fetch_params(w + 1);
                if (w >= 1) {
                    // the sub-tiles swept one anti-diagonal ago, carried into the sub-tiles two or more ahead of them
                    const int first = w + 1 - ap > 0 ? w + 1 - ap : 0;
                    for (int bp = first; bp < NSUB; ++bp) carry_into(Ys, Cs, LUs, ap, bp, w - 1 - bp, w - 1 - ap, lane);
                    __syncwarp();
                }
                if constexpr (PUSH) {
                    const bool pvec = n % 4 == 0 && reinterpret_cast<uintptr_t>(yng) % (4 * sizeof(F)) == 0;
                    if (owes_down && w == 1) {  // the strip of L[I + 1, I]: first used three anti-diagonals from here
                        const int64_t gi = i0 + TILE + ap * SUB + (lane >> 2) * 2;
                        const bool lvec = m % 4 == 0 && reinterpret_cast<uintptr_t>(lg) % (4 * sizeof(F)) == 0;
#pragma unroll
                        for (int as = 0; as < NSUB; ++as) {
                            const int64_t col = i0 + as * SUB + (lane & 3) * 4;
                            F t0[4] = {(F)0, (F)0, (F)0, (F)0}, t1[4] = {(F)0, (F)0, (F)0, (F)0};
                            if (lvec) {
                                if (gi < m) load4(lg + gi * m + col, t0);
                                if (gi + 1 < m) load4(lg + (gi + 1) * m + col, t1);
                            } else {
#pragma unroll
                                for (int x = 0; x < 4; ++x) {
                                    if (gi < m) t0[x] = lg[gi * m + col + x];
                                    if (gi + 1 < m) t1[x] = lg[(gi + 1) * m + col + x];
                                }
                            }
#pragma unroll
                            for (int x = 0; x < 4; ++x) { lb0[as * 4 + x] = t0[x]; lb1[as * 4 + x] = t1[x]; }
                        }
                    }
                    if (owes_right && w >= 1) {
                        // right push: the completed C of the row's sub-tile swept one anti-diagonal ago times its block
                        // row of U[J, J + 1]; a row is stored once its last sub-tile has gone in
                        const int b = w - 1 - ap;
                        if (ap < NSUB - 1 && b >= 0 && b < NSUB) {
#pragma unroll
                            for (int cb = 0; cb < NSUB; ++cb) mm16_acc(yn0[cb], yn1[cb], Cs + ap * SUB * LD + b * SUB, Ubs + b * SUB * LD + cb * SUB, lane);
                            if (b == NSUB - 1) {
#pragma unroll
                                for (int cb = 0; cb < NSUB; ++cb)
                                    store_block(yng + (i0 + ap * SUB) * n + j0 + TILE + cb * SUB, n, yn0[cb], yn1[cb], lane, m - (i0 + ap * SUB), n - (j0 + TILE + cb * SUB), pvec);
                            }
                        }
                        const int b3 = w - NSUB;  // the last row's sub-tile swept one anti-diagonal ago: this helper's column block of it
                        if (b3 >= 0 && b3 < NSUB) mm16_acc(y30, y31, Cs + (NSUB - 1) * SUB * LD + b3 * SUB, Ubs + b3 * SUB * LD + ap * SUB, lane);
                    }
                    if (owes_down) {
                        // down push: a column of sub-tiles is complete three anti-diagonals after its first; this helper's
                        // row strip of L[I + 1, I] times the column's errors, stored at once
                        const int b = w - NSUB;
                        if (b >= 0) {
                            F d0[4] = {(F)0, (F)0, (F)0, (F)0}, d1[4] = {(F)0, (F)0, (F)0, (F)0};
#pragma unroll
                            for (int as = 0; as < NSUB; ++as) mm16_areg(d0, d1, lb0 + as * 4, lb1 + as * 4, Ys + as * SUB * LD + b * SUB, lane);
                            store_block(cng + (i0 + TILE + ap * SUB) * n + j0 + b * SUB, n, d0, d1, lane, m - (i0 + TILE + ap * SUB), n - (j0 + b * SUB), pvec);
                        }
                        if (!more) {  // the last column, up to the term of the sub-tile being swept now
#pragma unroll
                            for (int as = 0; as < NSUB - 1; ++as) mm16_areg(c30, c31, lb0 + as * 4, lb1 + as * 4, Ys + as * SUB * LD + (NSUB - 1) * SUB, lane);
                        }
                    }
                }
                if (more) finish_params();
                __syncthreads();
                {   // the rounded values of the sub-tiles just swept: helper warp ap writes out the block of its row
                    const int bz = w - ap;
                    if (bz >= 0 && bz < NSUB) {
                        const bool zvec = n % 4 == 0 && reinterpret_cast<uintptr_t>(yg) % (4 * sizeof(F)) == 0;
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const int e = lane * 2 + q, row = e >> 2, c4 = (e & 3) * 4;
                            const int64_t gi = i0 + ap * SUB + row, gj = j0 + bz * SUB + c4;
                            F v[4];
                            load4(Zst + (ap * SUB + row) * ZLD + c4, v);
                            if (gi < m) {
                                if (zvec) {
                                    if (gj < n) store4(yg + gi * n + gj, v);
                                } else {
#pragma unroll
                                    for (int x = 0; x < 4; ++x)
                                        if (gj + x < n) yg[gi * n + gj + x] = v[x];
                                }
                            }
                        }
                    }
                }
                // ---- between two sweeps: the anti-diagonal just swept, carried into the next one; the next parameters ----
                if (more) {
                    store_params();
                    const int bn = w + 1 - ap;
                    if (bn >= 0 && bn < NSUB) carry_into(Ys, Cs, LUs, ap, bn, ap - 1, bn - 1, lane);
                    __syncthreads();
                }
            }
            // ---- neighbour push: the last sub-tile's terms, one product per helper and plane ----
            if constexpr (PUSH) {
                {
                    const bool pvec = n % 4 == 0 && reinterpret_cast<uintptr_t>(yng) % (4 * sizeof(F)) == 0;
                    const int x = helper, last = NSUB - 1;
                    if (owes_right) {
                        mm16_acc(y30, y31, Cs + last * SUB * LD + last * SUB, Ubs + last * SUB * LD + x * SUB, lane);
                        store_block(yng + (i0 + last * SUB) * n + j0 + TILE + x * SUB, n, y30, y31, lane, m - (i0 + last * SUB), n - (j0 + TILE + x * SUB), pvec);
                    }
                    if (owes_down) {
                        mm16_areg(c30, c31, lb0 + last * 4, lb1 + last * 4, Ys + last * SUB * LD + last * SUB, lane);
                        store_block(cng + (i0 + TILE + x * SUB) * n + j0 + last * SUB, n, c30, c31, lane, m - (i0 + TILE + x * SUB), n - (j0 + last * SUB), pvec);
                    }
                }
            }
        }
        // ---- operands of the tensor-core macro updates: tf32 hi / lo of E (transposed) and of the completed C ----
        if (P.c_hi != nullptr) {
            if constexpr (sizeof(F) == sizeof(float)) {
                auto split4 = [](const float (&v)[4], float (&hi)[4], float (&lo)[4]) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        uint32_t h;
                        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v[x]));
                        hi[x] = __uint_as_float(h);
                        lo[x] = v[x] - hi[x];
                    }
                };
                if (vec) {
                    // whole tile, rows of 16-byte multiples: four entries per thread and store.  C along its rows; E
                    // transposed: a thread gathers four rows of one column (consecutive threads take consecutive
                    // columns, so the shared-memory reads do not collide) and writes them as one vector of a row of E^T
                    for (int idx = tid; idx < TILE * TILE / 4; idx += TTH) {
                        {
                            const int r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                            float v[4], hi[4], lo[4];
                            load4(reinterpret_cast<const float *>(Cs) + r * LD + c, v);
                            split4(v, hi, lo);
                            store4(P.c_hi + (i0 + r) * n + j0 + c, hi);
                            store4(P.c_lo + (i0 + r) * n + j0 + c, lo);
                        }
                        {
                            const int c = idx % TILE, r = (idx / TILE) * 4;
                            float v[4], hi[4], lo[4];
#pragma unroll
                            for (int x = 0; x < 4; ++x) v[x] = (float)Ys[(r + x) * LD + c];
                            split4(v, hi, lo);
                            store4(P.et_hi + (j0 + c) * m + i0 + r, hi);
                            store4(P.et_lo + (j0 + c) * m + i0 + r, lo);
                        }
                    }
                } else {
                    for (int idx = tid; idx < TILE * TILE; idx += TTH) {
                        {   // C[i][j], consecutive threads along j
                            const int r = idx / TILE, c = idx % TILE;
                            const int64_t gi = i0 + r, gj = j0 + c;
                            if (gi < m && gj < n) {
                                const float v = (float)Cs[r * LD + c];
                                uint32_t h;
                                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
                                P.c_hi[gi * n + gj] = __uint_as_float(h);
                                P.c_lo[gi * n + gj] = v - __uint_as_float(h);
                            }
                        }
                        {   // E^T[j][i], consecutive threads along i
                            const int c = idx / TILE, r = idx % TILE;
                            const int64_t gi = i0 + r, gj = j0 + c;
                            if (gi < m && gj < n) {
                                const float v = (float)Ys[r * LD + c];
                                uint32_t h;
                                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
                                P.et_hi[gj * m + gi] = __uint_as_float(h);
                                P.et_lo[gj * m + gi] = v - __uint_as_float(h);
                            }
                        }
                    }
                }
            }
        }
        // ---- store the errors and the completed C of the tile ----
        if (vec) {
            for (int idx = tid; idx < TILE * TILE / 4; idx += TTH) {
                const int r = idx / (TILE / 4), c = (idx % (TILE / 4)) * 4;
                F ve[4], vc[4];
                load4(Ys + r * LD + c, ve);
                load4(Cs + r * LD + c, vc);
                store4(eg + (i0 + r) * n + j0 + c, ve);
                store4(cg + (i0 + r) * n + j0 + c, vc);
            }
        } else {
            for (int idx = tid; idx < TILE * TILE; idx += TTH) {
                const int r = idx / TILE, c = idx % TILE;
                const int64_t gi = i0 + r, gj = j0 + c;
                if (gi < m && gj < n) {
                    eg[gi * n + gj] = Ys[r * LD + c];
                    cg[gi * n + gj] = Cs[r * LD + c];
                }
            }
        }
        __syncthreads();
    }
}

template <typename F, int KIND>
static int launch_kind(const SweepArgs<F> &args, int S, int parity, cudaStream_t stream) {
    // the opt-in to more than 48 KB of dynamic shared memory is per device
    static PerDeviceOnce configured;
    const size_t smem = sizeof(F) * (4 * TILE * LD + 2 * NSUB * DBLK + 3 * SUB * LANES + NSUB * SUB * ZLD) + sizeof(unsigned) * (2 * LANES + 2 * SWEEPERS);
    // and the largest shared-memory carve-out, like the update kernels that run on the neighbouring SMs
    if (configured.run([&] {
            return cudaFuncSetAttribute(tile_sweep_kernel<F, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
                   cudaFuncSetAttribute(tile_sweep_kernel<F, KIND>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) == cudaSuccess;
        }) != G2D_OK)
        return G2D_ERR_CUDA;
    const int i_lo = S - args.nJ + 1 > 0 ? S - args.nJ + 1 : 0;
    const int i_hi = S + 1 < args.nI ? S + 1 : args.nI;
    // parity 0: every tile of the anti-diagonal; 1: tiles with even row and column index; 2: odd row and column index
    int first = i_lo, step = 1, count = i_hi - i_lo;
    if (parity != 0) {
        const int want = parity == 1 ? 0 : 1;
        if ((S & 1) != 0) return G2D_OK;  // row + column parity is even for both selections
        first = i_lo + (((i_lo & 1) != want) ? 1 : 0);
        step = 2;
        count = first < i_hi ? (i_hi - first + 1) / 2 : 0;
    }
    if (count <= 0) return G2D_OK;
    dim3 grid((unsigned)count, (unsigned)(args.batch < 65535 ? args.batch : 65535));
    tile_sweep_kernel<F, KIND><<<grid, TTH, smem, stream>>>(args, S, first, step);
    return check_launch();
}

template <typename F>
int launch_tile_sweep(const SweepArgs<F> &args, int S, cudaStream_t stream, int parity) {
    switch (args.kind) {
    case G2D_Q_ROUND: return launch_kind<F, G2D_Q_ROUND>(args, S, parity, stream);
    case G2D_Q_AFFINE: return launch_kind<F, G2D_Q_AFFINE>(args, S, parity, stream);
    case G2D_Q_FORCED: return launch_kind<F, G2D_Q_FORCED>(args, S, parity, stream);
    default: return G2D_ERR_UNSUPPORTED;
    }
}

template int launch_tile_sweep<float>(const SweepArgs<float> &, int, cudaStream_t, int);
template int launch_tile_sweep<double>(const SweepArgs<double> &, int, cudaStream_t, int);

}  // namespace g2d
