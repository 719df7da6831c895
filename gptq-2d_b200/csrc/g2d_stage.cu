// Per-stage kernels of the generic path, where the caller's own quantizer runs between launches
// and must see live Y (gptq_2d.py:1395-1400 of the reference).
//
// stage_error_kernel : E = z - Y on the sources of stage s, C += E there (the completed C), Y = z.
// stage_push_kernel  : every entry of the stages s+1..s1-1 that lies below a source (same column band)
//                      or right of one (same row band) receives its push, down first, in one
//                      read-modify-write; a receiver has at most one source of each kind per stage.
// Together they do the work of _push_kernel + _add_own_errors_kernel (gptq_2d.py:243-409) and of
// _push_down_super_entry_kernel + _push_right_super_entry_kernel (:428-601).
#include "g2d_common.cuh"

namespace g2d {

template <typename F>
struct StageArgs {
    F *y, *c, *e;
    const F *l, *u, *z;
    const int64_t *l_off, *u_off;
    int64_t batch, m, n, s, s1;
    int p, q;
    // N-factor sweeps run their slabs as batches that are `skew[batch]` stages behind (null: none); z then holds
    // z_stride values per batch (0: the stage's own d p q)
    const int32_t *skew;
    int64_t z_stride;
};

template <typename F>
__global__ void stage_error_kernel(StageArgs<F> A) {
    const int64_t mbar = A.m / A.p, nbar = A.n / A.q;
    const int64_t pq = (int64_t)A.p * A.q;
    if (A.skew != nullptr) {
        // every batch at a stage of its own: z_stride values per batch, the first d p q of them in use
        const int64_t total = A.z_stride * A.batch;
        for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
            const int64_t batch = t / A.z_stride, rest = t % A.z_stride;
            const int64_t s = A.s - A.skew[batch];
            if (s < 0 || s >= mbar + nbar - 1) continue;
            const int64_t i_lo = max((int64_t)0, s - nbar + 1), i_hi = min(s + 1, mbar);
            const int64_t k = rest / pq;
            if (k >= i_hi - i_lo) continue;
            const int a = (int)(rest % pq) / A.q, b = (int)(rest % pq) % A.q;
            const int64_t i = (i_lo + k) * A.p + a, j = (s - i_lo - k) * A.q + b;
            const int64_t at = batch * A.m * A.n + i * A.n + j;
            const F zv = A.z[t];
            const F ev = zv - A.y[at];
            A.e[at] = ev;
            A.c[at] += ev;
            A.y[at] = zv;
        }
        return;
    }
    const int64_t i_lo = max((int64_t)0, A.s - nbar + 1), i_hi = min(A.s + 1, mbar);
    const int64_t d = i_hi - i_lo, per_batch = d * pq;
    const int64_t total = per_batch * A.batch;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t batch = t / per_batch, rest = t % per_batch;
        const int64_t k = rest / pq;
        const int a = (int)(rest % pq) / A.q, b = (int)(rest % pq) % A.q;
        const int64_t i = (i_lo + k) * A.p + a, j = (A.s - i_lo - k) * A.q + b;
        const int64_t at = batch * A.m * A.n + i * A.n + j;
        const F zv = A.z[batch * (A.z_stride ? A.z_stride : per_batch) + rest];
        const F ev = zv - A.y[at];
        A.e[at] = ev;
        A.c[at] += ev;
        A.y[at] = zv;
    }
}

template <typename F>
__global__ void stage_push_kernel(StageArgs<F> A) {
    const int64_t mbar = A.m / A.p, nbar = A.n / A.q;
    const int p = A.p, q = A.q;
    const int64_t pq = (int64_t)p * q;
    const int64_t dd = 1 + blockIdx.y;  // receivers on coarse anti-diagonal s + dd
    for (int64_t batch = blockIdx.z; batch < A.batch; batch += gridDim.z) {
        const int64_t s = A.s - (A.skew ? A.skew[batch] : 0), sr = s + dd;
        if (s < 0 || sr >= mbar + nbar - 1) continue;
        const int64_t r_lo = max((int64_t)0, sr - nbar + 1), r_hi = min(sr + 1, mbar);
        const int64_t count = (r_hi - r_lo) * pq;
        F *yg = A.y + batch * A.m * A.n, *cg = A.c + batch * A.m * A.n;
        const F *eg = A.e + batch * A.m * A.n;
        const F *lg = A.l + (A.l_off ? A.l_off[batch] : 0);
        const F *ug = A.u + (A.u_off ? A.u_off[batch] : 0);
        for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (int64_t)gridDim.x * blockDim.x) {
            const int64_t rb = r_lo + t / pq, cb = sr - rb;
            const int a = (int)(t % pq) / q, b = (int)(t % pq) % q;
            const int64_t i = rb * p + a, j = cb * q + b;
            F down = (F)0, right = (F)0;
            bool any = false;
            if (rb - dd >= 0) {  // source (rb - dd, cb) in the same column band
                const int64_t k0 = (rb - dd) * p;
                for (int x = 0; x < p; ++x) down += lg[i * A.m + k0 + x] * eg[(k0 + x) * A.n + j];
                any = true;
            }
            if (cb - dd >= 0) {  // source (rb, cb - dd) in the same row band, its C completed by stage_error_kernel
                const int64_t k0 = (cb - dd) * q;
                for (int x = 0; x < q; ++x) right += cg[i * A.n + k0 + x] * ug[(k0 + x) * A.n + j];
                any = true;
            }
            if (any) {
                if (rb - dd >= 0) cg[i * A.n + j] += down;
                yg[i * A.n + j] += down + right;
            }
        }
    }
}

template <typename F>
int launch_stage_push(const g2d_stage_desc &d, const F *z, int64_t s, int64_t s1, cudaStream_t stream, const int32_t *skew, int64_t z_stride) {
    StageArgs<F> A;
    A.skew = skew; A.z_stride = z_stride;
    A.y = (F *)d.y; A.c = (F *)d.c; A.e = (F *)d.e;
    A.l = (const F *)d.l; A.u = (const F *)d.u; A.z = z;
    A.l_off = d.l_offsets; A.u_off = d.u_offsets;
    A.batch = d.batch; A.m = d.m; A.n = d.n; A.s = s; A.s1 = s1;
    A.p = d.p; A.q = d.q;
    const int64_t mbar = d.m / d.p, nbar = d.n / d.q, stages = mbar + nbar - 1;
    if (skew == nullptr && (s < 0 || s >= stages)) return G2D_ERR_BAD_ARGUMENT;
    if (s1 <= s) return G2D_ERR_BAD_ARGUMENT;
    if (skew == nullptr && s1 > stages) s1 = stages;
    const int64_t i_lo = s - nbar + 1 > 0 ? s - nbar + 1 : 0, i_hi = s + 1 < mbar ? s + 1 : mbar;
    const int64_t total = skew != nullptr ? z_stride * d.batch : (i_hi - i_lo) * d.p * d.q * d.batch;
    if (total <= 0) return G2D_OK;
    {
        const int threads = 128;
        int64_t blocks = ceil_div(total, threads);
        if (blocks > 65535 * 16) blocks = 65535 * 16;
        stage_error_kernel<F><<<(unsigned)blocks, threads, 0, stream>>>(A);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    }
    const int64_t pushes = s1 - s - 1;
    if (pushes > 0) {
        const int64_t lanes = mbar < nbar ? mbar : nbar;
        const int threads = 128;
        int64_t bx = ceil_div(lanes * d.p * d.q, threads);
        if (bx > 4096) bx = 4096;
        dim3 grid((unsigned)bx, (unsigned)pushes, (unsigned)(d.batch < 65535 ? d.batch : 65535));
        if (pushes > 65535) return G2D_ERR_TOO_LARGE;
        stage_push_kernel<F><<<grid, threads, 0, stream>>>(A);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    }
    return G2D_OK;
}

template int launch_stage_push<float>(const g2d_stage_desc &, const float *, int64_t, int64_t, cudaStream_t, const int32_t *, int64_t);
template int launch_stage_push<double>(const g2d_stage_desc &, const double *, int64_t, int64_t, cudaStream_t, const int32_t *, int64_t);

}  // namespace g2d
