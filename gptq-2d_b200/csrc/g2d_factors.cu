// Factor preparation: the unit (block) lower triangular L with M^{-1} = L Lambda L^T for a symmetric positive
// definite M, i.e. ldl_of_inverse + _unit_diagonal_blocks of the reference (gptq_2d_reference.py:29-49), which
// there is torch.linalg.cholesky + solve_triangular.  Same three steps, blocked by 64 and written for the GPU:
//
//   1. reverse-order Cholesky  M = T^T T  (T lower triangular; T^T is the reference's upper factor Um), from the
//      last block row to the first: factor the diagonal block in one CTA (and invert it), solve the block row to
//      its left as a product with that inverse, subtract the block row's Gram from the part still to factor;
//   2. Lf = T^{-1} (= Um^{-T}) by block forward substitution, one block row per launch:
//      Lf[i, j] = -T[i, i]^{-1} sum_{k = j .. i-1} T[i, k] Lf[k, j],  Lf[i, i] = T[i, i]^{-1};
//   3. out = Lf D^{-1} with D the size x size diagonal blocks of Lf: identity diagonal blocks, zeros above.
//
// M is overwritten (its lower triangle becomes T).  A non-positive pivot stores its 1-based index in *flag.
#include <mutex>

#include <type_traits>

#include "g2d_common.cuh"

namespace g2d {

constexpr int FB = 64;        // block edge
constexpr int FK = 16;        // k chunk of the tile products
constexpr int FLD = FB + 4;   // shared row stride
constexpr int FTH = 64;       // threads of a tile-product CTA (8 x 8 outputs each)

__device__ __forceinline__ int own8(int t, int x) { return x < 4 ? t * 4 + x : 32 + t * 4 + (x - 4); }

// acc[8][8] += sum_{k < K} A(i, k) B(k, j) for the 64 x 64 tile of this CTA; la / lb return 0 outside the matrix.
template <typename F, typename LA, typename LB>
__device__ __forceinline__ void tile_product(F (&acc)[8][8], int64_t K, LA la, LB lb, F *As, F *Bs, bool a_k_contiguous) {
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
    for (int64_t k0 = 0; k0 < K; k0 += FK) {
        F ra[FB * FK / FTH], rb[FB * FK / FTH];
#pragma unroll
        for (int t = 0; t < FB * FK / FTH; ++t) {
            const int idx = t * FTH + tid;
            const int i = a_k_contiguous ? idx / FK : idx % FB, kk = a_k_contiguous ? idx % FK : idx / FB;
            ra[t] = k0 + kk < K ? la(i, k0 + kk) : (F)0;
            const int kb = idx / FB, j = idx % FB;
            rb[t] = k0 + kb < K ? lb(k0 + kb, j) : (F)0;
        }
        __syncthreads();  // the previous chunk has been consumed
#pragma unroll
        for (int t = 0; t < FB * FK / FTH; ++t) {
            const int idx = t * FTH + tid;
            const int i = a_k_contiguous ? idx / FK : idx % FB, kk = a_k_contiguous ? idx % FK : idx / FB;
            As[kk * FLD + i] = ra[t];
            Bs[(idx / FB) * FLD + idx % FB] = rb[t];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < FK; ++kk) {
            F a[8], b[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) a[x] = As[kk * FLD + own8(ty, x)];
#pragma unroll
            for (int y = 0; y < 8; ++y) b[y] = Bs[kk * FLD + own8(tx, y)];
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int y = 0; y < 8; ++y) acc[x][y] += a[x] * b[y];
        }
    }
    __syncthreads();
}

// Up to two factorizations advance together, block step by block step, in the same launches (the steps are chains of
// short dependent kernels, so a second matrix rides along almost for free).  Problem z of a launch is blockIdx.y, or
// folded into blockIdx.x where the grid is three-dimensional already.  Block rows are taken in groups of GROUP
// (the trailing update of a tensor-core problem is applied once per group), and the problems are lined up so that
// their groups end at the same steps: with block-row counts rounded up to a multiple of GROUP, the launch for block
// row s of the largest problem serves block row s - (steps - rounded count) of a smaller one.
constexpr int GROUP = 4;
template <typename F>
struct LdlProblem {
    F *a, *out, *tinv, *w;
    int64_t n;
    int *flag;
    int tc;                       // trailing updates of whole groups run on the tensor cores (float, n % 4 == 0)
    float *pt_hi[2], *pt_lo[2];   // [n][GROUP * 64] transposed split panels of the even and odd groups
};
template <typename F>
struct LdlBatch {
    LdlProblem<F> p[2];
    int count;
    int steps;  // block rows of the largest problem, rounded up to a multiple of GROUP
};
__host__ __device__ inline int padded_block_rows(int64_t n) { return (int)(ceil_div(ceil_div(n, (int64_t)64), (int64_t)GROUP) * GROUP); }
#define LDL_PROBLEM(z)                                        \
    const LdlProblem<F> Q = (z) ? B.p[1] : B.p[0];            \
    F *const a = Q.a;                                         \
    const int64_t n = Q.n;                                    \
    const int kb = step_down - (B.steps - padded_block_rows(n)); \
    if (kb < 0 || (int64_t)kb * FB >= n) return;

template <typename F>
__device__ __forceinline__ void zero_acc(F (&acc)[8][8]) {
#pragma unroll
    for (int x = 0; x < 8; ++x)
#pragma unroll
        for (int y = 0; y < 8; ++y) acc[x][y] = (F)0;
}

// ---- step 1a: factor the diagonal block kb (bs x bs), M_kk = T_kk^T T_kk, and invert T_kk ----
// One CTA of 16 x 16 threads; thread (ty, tx) keeps the entries (ty + 16 a, tx + 16 b) of the (symmetric) working
// block in registers.  Step j (last row first): the owners of row j publish it, then everyone subtracts row j's outer
// product, scaled by 1 / pivot, from its part of the leading j x j block.  Row j is never touched again, the rows
// alternate between two buffers, so one barrier per step is enough.  Rows scaled by 1 / sqrt(pivot) are the factor.
template <typename F>
__global__ void __launch_bounds__(256) ldl_diag_kernel(LdlBatch<F> B, int step_down) {
    LDL_PROBLEM(blockIdx.y)
    F *const tinv = Q.tinv;
    int *const flag = Q.flag;
    __shared__ F S[FB][FB + 1];   // the block as loaded (lower triangle), later T in the lower and V^T in the upper triangle
    __shared__ F rowbuf[2][FB];   // published rows of the even and odd steps
    __shared__ F piv[FB];         // pivots
    __shared__ F Vd[FB];          // diagonal of the inverse
    __shared__ F Wt[FB * FB / 4]; // intermediate product of a doubling level
    __shared__ int bad;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t o = (int64_t)kb * FB;
    const int bs = (int)min((int64_t)FB, n - o);
    if (tid == 0) bad = 0;
    for (int idx = tid; idx < FB * FB; idx += 256) {
        const int r = idx / FB, c = idx % FB;
        F v = (F)0;
        if (r < bs && c <= r) v = a[(o + r) * n + o + c];
        if (r >= bs && r == c) v = (F)1;  // identity beyond a ragged block: its steps change nothing and the inverse stays finite
        S[r][c] = v;
    }
    __syncthreads();
    F reg[FB / 16][FB / 16];
#pragma unroll
    for (int aa = 0; aa < FB / 16; ++aa)
#pragma unroll
        for (int bb = 0; bb < FB / 16; ++bb) {
            const int i1 = ty + 16 * aa, i2 = tx + 16 * bb;
            reg[aa][bb] = i1 >= i2 ? S[i1][i2] : S[i2][i1];
        }
#pragma unroll
    for (int j = FB - 1; j >= 0; --j) {
        if (ty == (j & 15)) {
#pragma unroll
            for (int bb = 0; bb < FB / 16; ++bb) rowbuf[j & 1][tx + 16 * bb] = reg[j / 16][bb];
        }
        __syncthreads();
        const F d2 = rowbuf[j & 1][j];
        if (tid == 0) {
            piv[j] = d2;
            if (j < bs && !(d2 > (F)0)) bad = j + 1;
        }
        const F inv_d2 = (F)1 / d2;
        F rb[FB / 16];
#pragma unroll
        for (int bb = 0; bb < FB / 16; ++bb) rb[bb] = rowbuf[j & 1][tx + 16 * bb];
#pragma unroll
        for (int aa = 0; aa < FB / 16; ++aa) {
            if (16 * aa < j) {  // known at compile time: later blocks of rows are final already
                const int i1 = ty + 16 * aa;
                const F f = rowbuf[j & 1][i1] * inv_d2;
#pragma unroll
                for (int bb = 0; bb < FB / 16; ++bb)
                    if (16 * bb < j && i1 < j && tx + 16 * bb < j) reg[aa][bb] -= f * rb[bb];
            }
        }
    }
    __syncthreads();
    if (tid < FB) Vd[tid] = (F)1 / sqrt(piv[tid]);  // 1 / T[r][r]
    __syncthreads();
#pragma unroll
    for (int aa = 0; aa < FB / 16; ++aa)
#pragma unroll
        for (int bb = 0; bb < FB / 16; ++bb) {
            const int i1 = ty + 16 * aa, i2 = tx + 16 * bb;
            if (i1 > i2) S[i1][i2] = reg[aa][bb] * Vd[i1];
            if (i1 == i2) S[i1][i1] = sqrt(piv[i1]);
        }
    __syncthreads();
    // Inverse V of the lower triangular T_kk.  The strict upper triangle of S is free, so V is kept transposed there
    // (V[r][c] = S[c][r] for r > c) with its diagonal in Vd.  First the four 16 x 16 diagonal blocks by forward
    // substitution (one thread per column), then two doubling levels, each completing pairs of finished blocks
    // [A^{-1} 0; X B^{-1}] with X = -B^{-1} (C A^{-1}) as two small products over all threads.
    if (tid < FB) {
        const int c = tid, end = (tid & ~15) + 16;
        for (int r = c + 1; r < end; ++r) {
            F acc = -S[r][c] * Vd[c];
#pragma unroll 4
            for (int k = c + 1; k < r; ++k) acc -= S[r][k] * S[c][k];
            S[c][r] = acc * Vd[r];
        }
    }
    __syncthreads();
    for (int b = 16; b < FB; b *= 2) {
        const int outputs = (FB / (2 * b)) * b * b;
        for (int idx = tid; idx < outputs; idx += 256) {  // W = C A^{-1}, C = T[second half rows][first half columns]
            const int p = idx / (b * b), i = (idx / b) % b, j = idx % b, r0 = p * 2 * b, r1 = r0 + b;
            F acc = S[r1 + i][r0 + j] * Vd[r0 + j];
#pragma unroll 4
            for (int k = j + 1; k < b; ++k) acc += S[r1 + i][r0 + k] * S[r0 + j][r0 + k];
            Wt[idx] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < outputs; idx += 256) {  // X = -B^{-1} W, stored transposed
            const int p = idx / (b * b), i = (idx / b) % b, j = idx % b, r0 = p * 2 * b, r1 = r0 + b;
            F acc = Vd[r1 + i] * Wt[idx];
#pragma unroll 4
            for (int k = 0; k < i; ++k) acc += S[r1 + k][r1 + i] * Wt[(p * b + k) * b + j];
            S[r0 + j][r1 + i] = -acc;
        }
        __syncthreads();
    }
    for (int idx = tid; idx < FB * FB; idx += 256) {
        const int r = idx / FB, c = idx % FB;
        tinv[(int64_t)kb * FB * FB + idx] = (r < bs && c < bs && r >= c) ? (r == c ? Vd[r] : S[c][r]) : (F)0;
    }
    for (int idx = tid; idx < FB * FB; idx += 256) {
        const int r = idx / FB, c = idx % FB;
        if (r < bs && c < bs && r >= c) a[(o + r) * n + o + c] = S[r][c];
    }
    if (tid == 0 && bad && flag) atomicCAS(flag, 0, (int)(o + bad));
}

// ---- step 1b: block row to the left of the diagonal block: T[kb, j] = T_kk^{-T} M'[kb, j] ----
template <typename F>
__global__ void __launch_bounds__(FTH) ldl_trsm_kernel(LdlBatch<F> B, int step_down) {
    LDL_PROBLEM(blockIdx.y)
    const F *const tinv = Q.tinv;
    if ((int)blockIdx.x >= kb) return;
    __shared__ __align__(16) F As[FK * FLD];
    __shared__ __align__(16) F Bs[FK * FLD];
    const int j = blockIdx.x;  // column tile, j < kb
    const int64_t o = (int64_t)kb * FB, c0 = (int64_t)j * FB;
    const int bs = (int)min((int64_t)FB, n - o);
    const F *ti = tinv + (int64_t)kb * FB * FB;
    F acc[8][8];
    zero_acc(acc);
    // A(r, k) = Tinv[k][r] (transposed), B(k, col) = M'[o + k][c0 + col]
    tile_product<F>(acc, bs, [&](int r, int64_t k) { return ti[k * FB + r]; },
                    [&](int64_t k, int col) { return a[(o + k) * n + c0 + col]; }, As, Bs, false);
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        const int r = own8(ty, x);
#pragma unroll
        for (int y = 0; y < 8; ++y)
            if (r < bs) a[(o + r) * n + c0 + own8(tx, y)] = acc[x][y];
    }
    if constexpr (std::is_same<F, float>::value) {
        // tensor-core problems: the finished block row, transposed and split, is an operand of the group's trailing
        // update (columns left of the group only); rows beyond a ragged block are zero in acc already
        const int kb_lo = kb / GROUP * GROUP;
        if (Q.tc && j < kb_lo) {
            float *hi = Q.pt_hi[(kb / GROUP) & 1], *lo = Q.pt_lo[(kb / GROUP) & 1];
            const int k0 = (kb - kb_lo) * FB;
#pragma unroll
            for (int y = 0; y < 8; ++y) {
                const int64_t c = c0 + own8(tx, y);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float4 h, l;
                    split_tf32(acc[4 * half][y], h.x, l.x);
                    split_tf32(acc[4 * half + 1][y], h.y, l.y);
                    split_tf32(acc[4 * half + 2][y], h.z, l.z);
                    split_tf32(acc[4 * half + 3][y], h.w, l.w);
                    const int64_t at = c * (GROUP * FB) + k0 + own8(ty, 4 * half);
                    *reinterpret_cast<float4 *>(hi + at) = h;
                    *reinterpret_cast<float4 *>(lo + at) = l;
                }
            }
        }
    }
}

// ---- step 1c: M'[TI, TJ] -= T[kb, TI]^T T[kb, TJ] for TJ <= TI < kb (lower triangle of tiles) ----
template <typename F>
__global__ void __launch_bounds__(FTH) ldl_syrk_kernel(LdlBatch<F> B, int step_down) {
    LDL_PROBLEM(blockIdx.y)
    // tile pairs (TI, TJ), TJ <= TI < kb, in row order.  A tensor-core problem updates only the block rows of its own
    // group here (TI >= first block row of the group); the rows above wait for the group's update.
    const int kb_lo = Q.tc ? kb / GROUP * GROUP : 0;
    const int64_t first = (int64_t)kb_lo * (kb_lo + 1) / 2;
    if ((int64_t)blockIdx.x >= (int64_t)kb * (kb + 1) / 2 - first) return;
    __shared__ __align__(16) F As[FK * FLD];
    __shared__ __align__(16) F Bs[FK * FLD];
    // linear index -> (TI, TJ) with TJ <= TI
    const int64_t lin = first + blockIdx.x;
    int TI = (int)((sqrt(8.0 * (double)lin + 1.0) - 1.0) / 2.0);
    while ((int64_t)(TI + 1) * (TI + 2) / 2 <= lin) ++TI;
    while ((int64_t)TI * (TI + 1) / 2 > lin) --TI;
    const int TJ = (int)(lin - (int64_t)TI * (TI + 1) / 2);
    const int64_t o = (int64_t)kb * FB, r0 = (int64_t)TI * FB, c0 = (int64_t)TJ * FB;
    const int bs = (int)min((int64_t)FB, n - o);
    F acc[8][8];
    zero_acc(acc);
    tile_product<F>(acc, bs, [&](int i, int64_t k) { return a[(o + k) * n + r0 + i]; },
                    [&](int64_t k, int j) { return a[(o + k) * n + c0 + j]; }, As, Bs, false);
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        const int64_t r = r0 + own8(ty, x);
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            const int64_t c = c0 + own8(tx, y);
            if (c <= r) a[r * n + c] -= acc[x][y];
        }
    }
}

// ---- step 2: Lf = T^{-1} by doubling.  The 64 x 64 diagonal blocks of Lf are the inverted diagonal blocks of T.
// At level b (64, 128, ...) every aligned pair of finished b x b diagonal blocks [A^{-1} 0; . B^{-1}] is completed by
//     X = -B^{-1} (C A^{-1}),   C = T[second half rows, first half columns],
// as two batched tile products over all pairs: W = C A^{-1} into scratch, then X = -B^{-1} W into Lf.  Both inverses
// are lower triangular, which bounds the k range of every output tile. ----
template <typename F>
__global__ void __launch_bounds__(FTH) ldl_copy_diag_inverse_kernel(LdlBatch<F> B) {
    const LdlProblem<F> Q = blockIdx.y ? B.p[1] : B.p[0];
    const F *const tinv = Q.tinv;
    F *const out = Q.out;
    const int64_t n = Q.n;
    const int i = blockIdx.x;
    if ((int64_t)i * FB >= n) return;
    const int64_t r0 = (int64_t)i * FB;
    const int bs = (int)min((int64_t)FB, n - r0);
    for (int idx = threadIdx.x; idx < FB * FB; idx += FTH) {
        const int r = idx / FB, c = idx % FB;
        if (r < bs && c < bs) out[(r0 + r) * n + r0 + c] = tinv[(int64_t)i * FB * FB + idx];
    }
}

// second == false: W[pair block] = C A^{-1};  second == true: Lf[pair block] = -B^{-1} W
template <typename F>
__global__ void __launch_bounds__(FTH) ldl_trinv_level_kernel(LdlBatch<F> B, int64_t b, int pairs, bool second) {
    const LdlProblem<F> Q = (int)blockIdx.x >= pairs ? B.p[1] : B.p[0];
    const F *const a = Q.a;
    F *const w = Q.w, *const out = Q.out;
    const int64_t n = Q.n;
    __shared__ __align__(16) F As[FK * FLD];
    __shared__ __align__(16) F Bs[FK * FLD];
    const int64_t r0 = (int64_t)(blockIdx.x % pairs) * 2 * b, r1 = r0 + b;  // first half rows [r0, r1), second half rows [r1, r2)
    if (r1 >= n) return;
    const int64_t r2 = min(r0 + 2 * b, n);
    const int64_t ti = blockIdx.y, tj = blockIdx.z;  // output tile inside the b x b off-diagonal block
    const int64_t row0 = r1 + ti * FB, col0 = r0 + tj * FB;
    if (row0 >= r2) return;
    const int64_t rows = min((int64_t)FB, r2 - row0);
    F acc[8][8];
    zero_acc(acc);
    if (!second) {
        // W[i][j] = sum_{k >= j} C[i][k] A^{-1}[k][j]: k from the output tile's first column to the end of the first half
        const int64_t k_lo = col0, K = r1 - col0;
        tile_product<F>(acc, K, [&](int r, int64_t k) { return r < rows ? a[(row0 + r) * n + k_lo + k] : (F)0; },
                        [&](int64_t k, int c) { return out[(k_lo + k) * n + col0 + c]; }, As, Bs, true);
    } else {
        // X[i][j] = -sum_{k <= i} B^{-1}[i][k] W[k][j]: k from the start of the second half through the output tile's rows
        const int64_t k_lo = r1, K = min(row0 + FB, r2) - r1;
        tile_product<F>(acc, K, [&](int r, int64_t k) { return r < rows ? out[(row0 + r) * n + k_lo + k] : (F)0; },
                        [&](int64_t k, int c) { return w[(k_lo + k) * n + col0 + c]; }, As, Bs, true);
    }
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
    F *dst = second ? out : w;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        const int r = own8(ty, x);
#pragma unroll
        for (int y = 0; y < 8; ++y)
            if (r < rows) dst[(row0 + r) * n + col0 + own8(tx, y)] = second ? -acc[x][y] : acc[x][y];
    }
}

// ---- step 3: out = Lf D^{-1}.  Everything above the diagonal blocks is zero already (the output starts as zeros and
// only blocks on and below the diagonal are written), so the normalisation proper only sets the diagonal blocks to the
// identity: one thread per row ----
template <typename F>
__global__ void ldl_normalize_kernel(F *out, int64_t n, int size) {
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < n; row += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c0 = row / size * size;
        F *p = out + row * n + c0;
        for (int x = 0; x < size; ++x) p[x] = c0 + x == row ? (F)1 : (F)0;
    }
}

// The normalisation reads the diagonal blocks while other rows are rewritten, so the blocks are copied out first.
template <typename F>
__global__ void ldl_copy_diag_kernel(const F *out, int64_t n, int size, F *dblk) {
    const int64_t total = (n / size) * size * size;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / ((int64_t)size * size);
        const int r = (int)(t / size % size), c = (int)(t % size);
        dblk[t] = out[(b * size + r) * n + b * size + c];
    }
}

// One CTA walks rows, its threads the column blocks left of the row's diagonal block (no index divisions per entry).
template <typename F>
__global__ void ldl_scale_kernel(F *out, int64_t n, int size, const F *dblk) {
    for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
        const int64_t below = row / size;  // column blocks strictly left of the diagonal block
        for (int64_t b = threadIdx.x; b < below; b += blockDim.x) {
            F *p = out + row * n + b * size;
            const F *d = dblk + b * size * size;
            // x D = r with D lower triangular: back substitution from the last column of the block
            for (int x = size - 1; x >= 0; --x) {
                F acc = p[x];
                for (int x2 = x + 1; x2 < size; ++x2) acc -= p[x2] * d[x2 * size + x];
                p[x] = acc / d[x * size + x];
            }
        }
    }
}

// Side streams for the look-ahead of the trailing updates.  Calls take lanes round robin, so two factorizations that
// a caller runs concurrently on two streams do not share one.  Created on first use per device and kept.
struct SideLane {
    cudaStream_t stream = nullptr;
    cudaEvent_t panel[4] = {}, rest[4] = {};
};
static SideLane *acquire_side_lane() {
    static std::mutex mutex;
    static SideLane lanes[64][4];
    static unsigned next[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    SideLane *lane = &lanes[device][next[device]++ & 3];
    if (!lane->stream) {
        if (cudaStreamCreateWithFlags(&lane->stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        for (int k = 0; k < 4; ++k)
            if (cudaEventCreateWithFlags(&lane->panel[k], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&lane->rest[k], cudaEventDisableTiming) != cudaSuccess)
                return nullptr;
    }
    return lane;
}

template <typename F>
int ldl_run(int count, const int64_t *ns, F *const *as, const int *sizes, F *const *outs, int *flags, void *const *workspaces, cudaStream_t st) {
    LdlBatch<F> B;
    B.count = count;
    B.steps = 0;
    F *dblks[2] = {nullptr, nullptr};
    SyrkTcMaps pt_maps[2][2];
    int64_t n_max = 0;
    bool any_tc = false;
    for (int z = 0; z < count; ++z) {
        const int64_t n = ns[z];
        const int nb = (int)ceil_div(n, FB);
        F *tinv = (F *)workspaces[z];                             // [nb][64][64]
        dblks[z] = tinv + (int64_t)nb * FB * FB;                  // [n / size][size][size]
        LdlProblem<F> &P = B.p[z];
        P = LdlProblem<F>{as[z], outs[z], tinv, dblks[z] + n * (int64_t)FB /* [n][n] scratch of the doubling steps */, n,
                          flags ? flags + z : nullptr, 0, {nullptr, nullptr}, {nullptr, nullptr}};
        // float problems whose rows are 16-byte multiples use the tensor cores; the choice depends on the problem alone,
        // never on its partner in the batch, so that a pair gives the results of two single calls
        if (std::is_same<F, float>::value && n % 4 == 0) {
            float *base = (float *)P.w + 10 * n * n;  // behind the scratch and the nine planes of the triangular inverse
            for (int k = 0; k < 2; ++k) {
                P.pt_hi[k] = base + (2 * k) * n * (GROUP * FB);
                P.pt_lo[k] = base + (2 * k + 1) * n * (GROUP * FB);
                if (!syrk_tc_maps(&pt_maps[z][k], P.pt_hi[k], P.pt_lo[k], n)) return G2D_ERR_CUDA;
            }
            P.tc = 1;
            any_tc = true;
        }
        const int padded = padded_block_rows(n);
        B.steps = padded > B.steps ? padded : B.steps;
        n_max = n > n_max ? n : n_max;
        if (cudaMemsetAsync(outs[z], 0, sizeof(F) * (size_t)n * n, st) != cudaSuccess) return G2D_ERR_CUDA;
    }
    if (count == 1) B.p[1] = B.p[0];
    if (flags && cudaMemsetAsync(flags, 0, sizeof(int) * count, st) != cudaSuccess) return G2D_ERR_CUDA;
    // Each step factors one 64-row block row (last first): diagonal block, panel to its left, trailing update.  The
    // update of a step reaches every row above for an ordinary problem, but only the rows of the step's own group of
    // GROUP block rows for a tensor-core problem; the rows above the group get the whole group's update at once
    // (K = 256) from the tensor cores.  Look-ahead: that update is split into the rows of the next group (kept on the
    // caller's stream) and the rest (a side stream), so that the latency-bound kernels of the next group overlap the
    // bulk of the update.  rest(g) touches the groups <= g - 2: group g needs rest(g + 2) and older before its first
    // kernel (which also frees the panel planes that it reuses), and next(g) must follow rest(g + 1), whose targets
    // it shares (the order of the additions is fixed, hence the result).
    SideLane *lane = acquire_side_lane();
    if (!lane) return G2D_ERR_CUDA;
    bool rest_recorded[4] = {false, false, false, false};
    const int groups = B.steps / GROUP;
    auto wait_rest = [&](int g) {
        if (g < groups && rest_recorded[g & 3]) return cudaStreamWaitEvent(st, lane->rest[g & 3], 0) == cudaSuccess;
        return true;
    };
    for (int s = B.steps - 1; s >= 0; --s) {  // block row of the largest problem; smaller problems are lined up by groups
        const int g = s / GROUP;
        if (s % GROUP == GROUP - 1 && !wait_rest(g + 2)) return G2D_ERR_CUDA;
        ldl_diag_kernel<F><<<dim3(1, count), 256, 0, st>>>(B, s);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        if (s == 0) break;
        int64_t panel_tiles = 0, update_tiles = 0;
        for (int z = 0; z < count; ++z) {
            const int kb = s - (B.steps - padded_block_rows(ns[z]));
            if (kb <= 0 || (int64_t)kb * FB >= ns[z]) continue;
            const int kb_lo = B.p[z].tc ? kb / GROUP * GROUP : 0;
            const int64_t tiles = (int64_t)kb * (kb + 1) / 2 - (int64_t)kb_lo * (kb_lo + 1) / 2;
            panel_tiles = kb > panel_tiles ? kb : panel_tiles;
            update_tiles = tiles > update_tiles ? tiles : update_tiles;
        }
        if (panel_tiles > 0) {
            ldl_trsm_kernel<F><<<dim3((unsigned)panel_tiles, count), FTH, 0, st>>>(B, s);
            if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        }
        if (update_tiles > 0) {
            ldl_syrk_kernel<F><<<dim3((unsigned)update_tiles, count), FTH, 0, st>>>(B, s);
            if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        }
        if (s % GROUP != 0 || !any_tc) continue;
        // the group g is complete: its update of everything above, for the tensor-core problems
        SyrkTcTarget next[2], rest[2];
        int targets = 0;
        bool any_rest = false;
        for (int z = 0; z < count; ++z) {
            const int kb_lo = s - (B.steps - padded_block_rows(ns[z]));
            if (!B.p[z].tc || kb_lo <= 0) continue;
            const int64_t o = (int64_t)kb_lo * FB;
            const int t_all = (int)(o / 128), t_next = t_all - GROUP * FB / 128;  // tile rows above the group; those of the next group start at t_next
            const int kw = (int)(ns[z] - o < GROUP * FB ? ns[z] - o : GROUP * FB);
            SyrkTcTarget t{&pt_maps[z][(kb_lo / GROUP) & 1], B.p[z].pt_hi[(kb_lo / GROUP) & 1], B.p[z].pt_lo[(kb_lo / GROUP) & 1],
                           (float *)B.p[z].a, ns[z], t_next, t_all, kw, B.p[z].flag};
            next[targets] = t;
            t.t_lo = 0;
            t.t_hi = t_next;
            rest[targets] = t;
            any_rest = any_rest || t_next > 0;
            ++targets;
        }
        if (targets == 0) continue;
        rest_recorded[g & 3] = false;
        if (any_rest) {  // the panels are final: the side stream may start on the rows above the next group
            if (cudaEventRecord(lane->panel[g & 3], st) != cudaSuccess || cudaStreamWaitEvent(lane->stream, lane->panel[g & 3], 0) != cudaSuccess)
                return G2D_ERR_CUDA;
            const int status = launch_syrk_tc(targets, rest, lane->stream);
            if (status != G2D_OK) return status;
            if (cudaEventRecord(lane->rest[g & 3], lane->stream) != cudaSuccess) return G2D_ERR_CUDA;
        }
        if (!wait_rest(g + 1)) return G2D_ERR_CUDA;
        const int status = launch_syrk_tc(targets, next, st);
        if (status != G2D_OK) return status;
        rest_recorded[g & 3] = any_rest;
    }
    // everything the side stream did joins the caller's stream before the inverse starts
    for (int k = 0; k < 4; ++k)
        if (rest_recorded[k] && cudaStreamWaitEvent(st, lane->rest[k], 0) != cudaSuccess) return G2D_ERR_CUDA;
    ldl_copy_diag_inverse_kernel<F><<<dim3(B.steps, count), FTH, 0, st>>>(B);
    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    // The 64-level for everyone; from the 128-level on, float problems whose rows are 16-byte multiples continue on the
    // tensor cores and the others here.  The choice depends on the problem alone, never on its partner in the batch.
    auto ffma_levels = [&](const LdlBatch<F> &batch, int problems, int64_t n_top, int64_t b_first, int64_t b_end) {
        for (int64_t b = b_first; b < n_top && b < b_end; b *= 2) {
            const int64_t pairs = ceil_div(n_top, 2 * b), tiles = b / FB;
            if (tiles > 65535) return (int)G2D_ERR_TOO_LARGE;
            dim3 grid((unsigned)(pairs * problems), (unsigned)tiles, (unsigned)tiles);
            ldl_trinv_level_kernel<F><<<grid, FTH, 0, st>>>(batch, b, (int)pairs, false);
            if (check_launch() != G2D_OK) return (int)G2D_ERR_CUDA;
            ldl_trinv_level_kernel<F><<<grid, FTH, 0, st>>>(batch, b, (int)pairs, true);
            if (check_launch() != G2D_OK) return (int)G2D_ERR_CUDA;
        }
        return (int)G2D_OK;
    };
    int status = ffma_levels(B, count, n_max, FB, 2 * FB);
    if (status != G2D_OK) return status;
    FactorPlanes planes[2];
    int tensor_count = 0;
    LdlBatch<F> rest = B;
    int rest_count = 0;
    int64_t rest_max = 0;
    for (int z = 0; z < count; ++z) {
        const int64_t n = ns[z];
        if (std::is_same<F, float>::value && n % 4 == 0) {
            float *base = (float *)B.p[z].w + n * n;  // nine [n][n] planes behind the scratch of the 64-level
            planes[tensor_count++] = FactorPlanes{(const float *)as[z], (float *)outs[z], base, base + n * n, base + 2 * n * n,
                                                  base + 3 * n * n, base + 4 * n * n, base + 5 * n * n, base + 6 * n * n, base + 7 * n * n,
                                                  base + 8 * n * n, n, flags ? flags + z : nullptr};
        } else {
            rest.p[rest_count++] = B.p[z];
            rest_max = n > rest_max ? n : rest_max;
        }
    }
    if (rest_count == 1) rest.p[1] = rest.p[0];
    if (rest_count > 0) {
        status = ffma_levels(rest, rest_count, rest_max, 2 * FB, INT64_MAX);
        if (status != G2D_OK) return status;
    }
    if (tensor_count > 0) {
        status = launch_trinv_tc(tensor_count, planes, st);
        if (status != G2D_OK) return status;
    }
    for (int z = 0; z < count; ++z) {
        const int64_t n = ns[z];
        const int size = sizes[z];
        const int64_t blocks = n < 148 * 16 ? n : 148 * 16;  // rows are dealt out to CTAs
        ldl_copy_diag_kernel<F><<<(unsigned)(ceil_div(n * size, 256) < 148 * 64 ? ceil_div(n * size, 256) : 148 * 64), 256, 0, st>>>(outs[z], n, size, dblks[z]);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        ldl_scale_kernel<F><<<(unsigned)blocks, 256, 0, st>>>(outs[z], n, size, dblks[z]);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        ldl_normalize_kernel<F><<<(unsigned)ceil_div(n, (int64_t)256), 256, 0, st>>>(outs[z], n, size);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    }
    return G2D_OK;
}

}  // namespace g2d

using namespace g2d;

static size_t ldl_bytes(int dtype, int64_t n) {
    const size_t elem = dtype == G2D_F32 ? 4 : 8;
    const size_t nb = (size_t)ceil_div(n, FB);
    // float: nine operand planes of the tensor-core triangular inverse and two pairs of transposed split panels
    const size_t planes = dtype == G2D_F32 ? 9 * (size_t)n * n + 4 * (size_t)n * GROUP * FB : 0;
    return ((nb * FB * FB + (size_t)n * FB + (size_t)n * n + planes) * elem + 255) & ~(size_t)255;
}

extern "C" int g2d_ldl_workspace_bytes(int dtype, int64_t n, size_t *bytes) {
    if ((dtype != G2D_F32 && dtype != G2D_F64) || n < 0 || !bytes) return G2D_ERR_BAD_ARGUMENT;
    *bytes = ldl_bytes(dtype, n);
    return G2D_OK;
}

static int ldl_check(int dtype, int64_t n, int32_t size, const void *a, const void *out, const void *workspace, size_t workspace_bytes) {
    if ((dtype != G2D_F32 && dtype != G2D_F64) || n <= 0 || size <= 0) return G2D_ERR_BAD_ARGUMENT;
    if (n % size != 0 || size > FB) return size > FB ? G2D_ERR_TOO_LARGE : G2D_ERR_BAD_ARGUMENT;
    if (!a || !out) return G2D_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < ldl_bytes(dtype, n)) return G2D_ERR_WORKSPACE;
    if (ceil_div(n, FB) > 46000) return G2D_ERR_TOO_LARGE;  // tile pairs of one launch must fit a 1-D grid
    return G2D_OK;
}

extern "C" int g2d_ldl_of_inverse(int dtype, int64_t n, void *a, int32_t size, void *out, int32_t *status_flag, void *workspace,
                                  size_t workspace_bytes, void *stream) {
    if (n == 0 && (dtype == G2D_F32 || dtype == G2D_F64) && size > 0) return G2D_OK;
    const int status = ldl_check(dtype, n, size, a, out, workspace, workspace_bytes);
    if (status != G2D_OK) return status;
    cudaStream_t st = (cudaStream_t)stream;
    const int sizes[1] = {size};
    void *const ws[1] = {workspace};
    if (dtype == G2D_F32) {
        float *as[1] = {(float *)a}, *outs[1] = {(float *)out};
        return ldl_run<float>(1, &n, as, sizes, outs, status_flag, ws, st);
    }
    double *as[1] = {(double *)a}, *outs[1] = {(double *)out};
    return ldl_run<double>(1, &n, as, sizes, outs, status_flag, ws, st);
}

extern "C" int g2d_ldl_of_inverse_pair(int dtype, int64_t n0, void *a0, int32_t size0, void *out0, void *workspace0, size_t workspace0_bytes,
                                       int64_t n1, void *a1, int32_t size1, void *out1, void *workspace1, size_t workspace1_bytes,
                                       int32_t *status_flags, void *stream) {
    int status = ldl_check(dtype, n0, size0, a0, out0, workspace0, workspace0_bytes);
    if (status != G2D_OK) return status;
    status = ldl_check(dtype, n1, size1, a1, out1, workspace1, workspace1_bytes);
    if (status != G2D_OK) return status;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t ns[2] = {n0, n1};
    const int sizes[2] = {size0, size1};
    void *const ws[2] = {workspace0, workspace1};
    if (dtype == G2D_F32) {
        float *as[2] = {(float *)a0, (float *)a1}, *outs[2] = {(float *)out0, (float *)out1};
        return ldl_run<float>(2, ns, as, sizes, outs, status_flags, ws, st);
    }
    double *as[2] = {(double *)a0, (double *)a1}, *outs[2] = {(double *)out0, (double *)out1};
    return ldl_run<double>(2, ns, as, sizes, outs, status_flags, ws, st);
}
