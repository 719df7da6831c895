// Super-entry and N-factor sweeps with the quantizer inside the library.
//
// The reference drives a super-entry sweep from Python: per coarse anti-diagonal it calls the quantizer (for the trellis
// code 2 x 129 kernel launches, quantizer_trellis.py:271-341) and the two super-entry push kernels
// (gptq_2d.py:428-601), and flushes at block ends (gptq_2d.py:1342-1374).  Here the whole loop runs inside one C call:
// per coarse stage a quantizer kernel of this library (round, affine, dynamic abs-max, trellis), the commit-and-push
// kernels and, at block ends, the band update.  Nothing returns to the host between stages, so a sweep is one
// asynchronous enqueue and can be captured.
//
// N-factor sweeps (Algorithm 4, gptq_2d_reference.py:269-294) run on the same loop.  A tensor [n_1, ..., n_D] with one
// unit lower triangular factor per mode is taken as a batch of n_1 ... n_{D-2} slabs [n_{D-1}, n_D]; slab b with the
// leading multi-index (i_1, ..., i_{D-2}) is a two-sided sweep under (L_{D-1}, L_D^T) whose input is
//     X_b + sum_k sum_{i' < i_k} L_k[i_k, i'] F_k[b with i_k -> i'],        F_k = Z - X - (the folds of the modes 0..k),
// because folding the errors of a finished slab through every remaining mode gives exactly Z - (its input): the
// leading modes couple the slabs by plain scaled additions of those residuals, entry by entry, and are never expanded
// into a Kronecker product.  An entry of slab b needs the same entry of the slabs before it in every leading mode,
// so slab b runs sigma_b = i_1 + ... + i_{D-2} stages behind slab 0: global stage g holds the hyper-anti-diagonal
// i_1 + ... + i_D = g, as in the reference, 1 + sum_d (n_d - 1) stages in all.
#include "g2d_common.cuh"

#include <vector>

namespace g2d {

namespace {

constexpr int MAX_LEAD = 4;

struct LeadModes {
    int count;
    int64_t size[MAX_LEAD], stride[MAX_LEAD];  // stride: batches per step of the mode's index
    const void *factor[MAX_LEAD];
};

template <typename F>
struct SuperArgs {
    F *y, *z;
    const F *scale, *zero;
    const int64_t *scale_off, *zero_off;
    int64_t srs, scs, zrs, zcs;
    F qmin, qmax, divisor;
    int half;
    const int32_t *skew;
    int64_t batch, m, n, stage, dmax;  // dmax: super-entries per batch that z holds at this stage
    int p, q;
    F *xs, *row_scale;                 // trellis: gathered sequences and their scales
    LeadModes lead;
    F *fold;                           // lead.count planes [batch, m, n]
};

// Entry (k, a, b) of the stage of `batch`: false when the batch has no such entry at this global stage.
template <typename F>
__device__ __forceinline__ bool locate(const SuperArgs<F> &A, int64_t batch, int64_t k, int a, int b, int64_t &i, int64_t &j) {
    const int64_t mbar = A.m / A.p, nbar = A.n / A.q;
    const int64_t s = A.stage - (A.skew ? A.skew[batch] : 0);
    if (s < 0 || s >= mbar + nbar - 1) return false;
    const int64_t i_lo = max((int64_t)0, s - nbar + 1), i_hi = min(s + 1, mbar);
    if (k >= i_hi - i_lo) return false;
    i = (i_lo + k) * A.p + a;
    j = (s - i_lo - k) * A.q + b;
    return true;
}

// One thread per entry of the stage: the leading modes' feedback is added to live Y, and the running fold planes are
// brought up to "minus the input of this entry's sub-problem at level k" (they started as -X).
template <typename F>
__global__ void fold_kernel(SuperArgs<F> A) {
    const int64_t pq = (int64_t)A.p * A.q, per = A.dmax * pq, total = per * A.batch, plane = A.batch * A.m * A.n;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t batch = t / per, rest = t % per;
        int64_t i, j;
        if (!locate(A, batch, rest / pq, (int)(rest % pq) / A.q, (int)(rest % pq) % A.q, i, j)) continue;
        const int64_t pos = i * A.n + j, at = batch * A.m * A.n + pos;
        F sum = (F)0;
        for (int k = 0; k < A.lead.count; ++k) {
            const int64_t size = A.lead.size[k], stride = A.lead.stride[k];
            const int64_t ik = batch / stride % size;
            const F *factor = (const F *)A.lead.factor[k] + ik * size;
            const F *residual = A.fold + (int64_t)k * plane + (batch - ik * stride) * A.m * A.n + pos;  // index 0 of mode k
            F fold = (F)0;
            for (int64_t ip = 0; ip < ik; ++ip) fold += factor[ip] * residual[ip * stride * A.m * A.n];
            sum += fold;
            A.fold[(int64_t)k * plane + at] -= sum;
        }
        A.y[at] += sum;
    }
}

// After the stage is rounded: F_k = Z - (input of the level-k sub-problem).
template <typename F>
__global__ void fold_commit_kernel(SuperArgs<F> A) {
    const int64_t pq = (int64_t)A.p * A.q, per = A.dmax * pq, total = per * A.batch, plane = A.batch * A.m * A.n;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t batch = t / per, rest = t % per;
        int64_t i, j;
        if (!locate(A, batch, rest / pq, (int)(rest % pq) / A.q, (int)(rest % pq) % A.q, i, j)) continue;
        const int64_t at = batch * A.m * A.n + i * A.n + j;
        const F zv = A.z[t];
        for (int k = 0; k < A.lead.count; ++k) A.fold[(int64_t)k * plane + at] += zv;
    }
}

template <typename F>
__global__ void negate_into_planes_kernel(const F *__restrict__ x, F *__restrict__ planes, int64_t count, int copies) {
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (int64_t)gridDim.x * blockDim.x) {
        const F v = -x[t];
        for (int k = 0; k < copies; ++k) planes[(int64_t)k * count + t] = v;
    }
}

__global__ void skew_kernel(int32_t *skew, int64_t batch, LeadModes lead) {
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < batch; b += (int64_t)gridDim.x * blockDim.x) {
        int64_t sum = 0;
        for (int k = 0; k < lead.count; ++k) sum += b / lead.stride[k] % lead.size[k];
        skew[b] = (int32_t)sum;
    }
}

// Elementwise quantizers of one stage (round, affine) and the gather of the trellis sequences: one thread per entry.
template <typename F, int KIND>
__global__ void quantize_entries_kernel(SuperArgs<F> A) {
    const int64_t pq = (int64_t)A.p * A.q, per = A.dmax * pq, total = per * A.batch;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t batch = t / per, rest = t % per;
        int64_t i, j;
        const bool on = locate(A, batch, rest / pq, (int)(rest % pq) / A.q, (int)(rest % pq) % A.q, i, j);
        if (KIND == G2D_Q_TRELLIS) {
            // sequences of super-entries that do not exist at this stage are searched along with the others (their result
            // is never read): give them zeros
            const F sc = A.scale[A.scale_off ? A.scale_off[batch] : 0];
            A.xs[t] = on ? div_rn(A.y[batch * A.m * A.n + i * A.n + j], sc) : (F)0;
            if (rest % pq == 0) A.row_scale[t / pq] = sc;
            continue;
        }
        if (!on) continue;
        const F yv = A.y[batch * A.m * A.n + i * A.n + j];
        if (KIND == G2D_Q_ROUND) {
            A.z[t] = rint_even(yv);
        } else {
            const F sc = A.scale[(A.scale_off ? A.scale_off[batch] : 0) + i * A.srs + j * A.scs];
            const F zp = A.zero[(A.zero_off ? A.zero_off[batch] : 0) + i * A.zrs + j * A.zcs];
            A.z[t] = affine_value(yv, sc, zp, A.qmin, A.qmax);
        }
    }
}

// Dynamic abs-max rounding (quantizer_int.py:120-134, :407-439): one warp per row of a super-entry.
template <typename F>
__global__ void quantize_absmax_kernel(SuperArgs<F> A) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5, rows = A.batch * A.dmax * A.p;
    for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const int64_t batch = row / (A.dmax * A.p), k = row / A.p % A.dmax;
        const int a = (int)(row % A.p);
        int64_t i, j;
        if (!locate(A, batch, k, a, 0, i, j)) continue;
        const F *src = A.y + batch * A.m * A.n + i * A.n + j;
        F top = (F)0;
        for (int c = lane; c < A.q; c += 32) top = fmax(top, fabs(src[c]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = fmax(top, __shfl_xor_sync(0xffffffffu, top, o));
        const F s = absmax_scale_value(top, A.divisor, A.half);
        for (int c = lane; c < A.q; c += 32) {
            F t = rint_even(div_rn(src[c], s));
            t = t < A.qmin ? A.qmin : t;
            t = t > A.qmax ? A.qmax : t;
            A.z[row * A.q + c] = mul_rn(t, s);
        }
    }
}

// Packed trellis paths of one stage into the matrix-level array [batch, m / p, n / q, bytes].
template <typename F>
__global__ void scatter_codes_kernel(SuperArgs<F> A, const uint8_t *__restrict__ stage_codes, uint8_t *__restrict__ codes, int64_t bytes) {
    const int64_t per = A.dmax * bytes, total = per * A.batch, nbar = A.n / A.q, mbar = A.m / A.p;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t batch = t / per, k = t % per / bytes, byte = t % bytes;
        int64_t i, j;
        if (!locate(A, batch, k, 0, 0, i, j)) continue;
        codes[((batch * mbar + i / A.p) * nbar + j / A.q) * bytes + byte] = stage_codes[t];
    }
}

inline unsigned blocks_for(int64_t work, int threads) {
    int64_t blocks = ceil_div(work, threads);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return (unsigned)blocks;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Plan {
    size_t c, e, z, skew, fold, xs, row_scale, stage_codes, viterbi, total;
    int64_t lanes, stages2d, lead_total;
    int64_t code_bytes;
};

int make_plan(const g2d_super_desc *d, Plan *plan) {
    const size_t elem = d->dtype == G2D_F32 ? 4 : 8;
    const int64_t mbar = d->m / d->p, nbar = d->n / d->q;
    plan->lanes = mbar < nbar ? mbar : nbar;
    plan->stages2d = mbar + nbar - 1;
    plan->lead_total = 0;
    for (int k = 0; k < d->lead_count; ++k) plan->lead_total += d->lead_size[k] - 1;
    const size_t matrix = align256(elem * (size_t)(d->batch * d->m * d->n));
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t where = at; at += align256(bytes); return where; };
    plan->c = take(matrix);
    plan->e = take(matrix);
    plan->z = take(elem * (size_t)(d->batch * plan->lanes * d->p * d->q));
    plan->skew = take(d->lead_count > 0 ? sizeof(int32_t) * (size_t)d->batch : 0);
    plan->fold = take((size_t)d->lead_count * matrix);
    plan->xs = plan->row_scale = plan->stage_codes = plan->viterbi = at;
    plan->code_bytes = 0;
    if (d->quant_kind == G2D_Q_TRELLIS) {
        const int64_t rows = d->batch * plan->lanes;
        const int T = d->p * d->q;
        plan->xs = take(elem * (size_t)(rows * T));
        plan->row_scale = take(elem * (size_t)rows);
        plan->code_bytes = trellis_code_bytes(T, d->trellis_L, d->trellis_K, d->trellis_V, d->tail_biting);
        plan->stage_codes = take(d->codes ? (size_t)(rows * plan->code_bytes) : 0);
        plan->viterbi = take(trellis_scratch_bytes(d->dtype, rows, T, d->trellis_L, d->trellis_K, d->trellis_V));
    }
    plan->total = at;
    return G2D_OK;
}

int check_super(const g2d_super_desc *d) {
    if (!d) return G2D_ERR_BAD_ARGUMENT;
    if (d->dtype != G2D_F32 && d->dtype != G2D_F64) return G2D_ERR_BAD_ARGUMENT;
    if (d->batch < 0 || d->m < 0 || d->n < 0 || d->p <= 0 || d->q <= 0) return G2D_ERR_BAD_ARGUMENT;
    if (d->m % d->p || d->n % d->q) return G2D_ERR_BAD_ARGUMENT;
    if (d->lead_count < 0 || d->lead_count > MAX_LEAD) return G2D_ERR_BAD_ARGUMENT;
    int64_t slabs = 1;
    for (int k = 0; k < d->lead_count; ++k) {
        if (d->lead_size[k] <= 0) return G2D_ERR_BAD_ARGUMENT;
        slabs *= d->lead_size[k];
    }
    if (d->lead_count > 0 && slabs != d->batch) return G2D_ERR_BAD_ARGUMENT;
    switch (d->quant_kind) {
    case G2D_Q_ROUND: break;
    case G2D_Q_AFFINE:
    case G2D_Q_ABSMAX_DYNAMIC:
        if (!(d->qmin < d->qmax)) return G2D_ERR_BAD_ARGUMENT;
        break;
    case G2D_Q_TRELLIS: {
        const int V = d->trellis_V, K = d->trellis_K, L = d->trellis_L, T = d->p * d->q;
        if (V < 1 || V > 2 || K < 1 || K * V > 8 || L < K * V || L > 24 || T % V != 0) return G2D_ERR_BAD_ARGUMENT;
        if (d->codes && d->tail_biting && (int64_t)(T / V) * K * V < L) return G2D_ERR_UNSUPPORTED;
        break;
    }
    default: return G2D_ERR_UNSUPPORTED;
    }
    return G2D_OK;
}

template <typename F>
int sweep_super(const g2d_super_desc *d, const Plan &plan, cudaStream_t st) {
    char *ws = (char *)d->workspace;
    const int64_t count = d->batch * d->m * d->n;
    F *c = (F *)(ws + plan.c), *e = (F *)(ws + plan.e), *z = (F *)(ws + plan.z);
    int32_t *skew = d->lead_count > 0 ? (int32_t *)(ws + plan.skew) : nullptr;
    if (cudaMemsetAsync(c, 0, sizeof(F) * (size_t)count, st) != cudaSuccess) return G2D_ERR_CUDA;

    SuperArgs<F> A{};
    A.y = (F *)d->y; A.z = z;
    A.scale = (const F *)d->scale; A.zero = (const F *)d->zero;
    A.scale_off = d->scale_offsets; A.zero_off = d->zero_offsets;
    A.srs = d->scale_row_stride; A.scs = d->scale_col_stride; A.zrs = d->zero_row_stride; A.zcs = d->zero_col_stride;
    A.qmin = (F)d->qmin; A.qmax = (F)d->qmax;
    A.divisor = (F)((d->qmax - d->qmin) / 2);
    A.half = d->half;
    A.skew = skew;
    A.batch = d->batch; A.m = d->m; A.n = d->n; A.p = d->p; A.q = d->q;
    A.xs = (F *)(ws + plan.xs); A.row_scale = (F *)(ws + plan.row_scale);
    A.fold = (F *)(ws + plan.fold);
    A.lead.count = d->lead_count;
    int64_t stride = d->batch;
    for (int k = 0; k < d->lead_count; ++k) {
        stride /= d->lead_size[k];
        A.lead.size[k] = d->lead_size[k];
        A.lead.stride[k] = stride;
        A.lead.factor[k] = d->lead_factor[k];
    }
    if (d->lead_count > 0) {
        skew_kernel<<<blocks_for(d->batch, 256), 256, 0, st>>>(skew, d->batch, A.lead);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
        negate_into_planes_kernel<F><<<blocks_for(count, 256), 256, 0, st>>>((const F *)d->y, A.fold, count, d->lead_count);
        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
    }

    g2d_stage_desc sd{};
    sd.dtype = d->dtype; sd.p = d->p; sd.q = d->q;
    sd.batch = d->batch; sd.m = d->m; sd.n = d->n;
    sd.y = d->y; sd.c = c; sd.e = e;
    sd.l = d->l; sd.l_offsets = d->l_offsets; sd.u = d->u; sd.u_offsets = d->u_offsets;
    BandArgs<F> b;
    b.y = (F *)d->y; b.c = c; b.e = e; b.l = (const F *)d->l; b.u = (const F *)d->u; b.l_off = d->l_offsets; b.u_off = d->u_offsets;
    b.batch = d->batch; b.m = d->m; b.n = d->n; b.P = d->p; b.Q = d->q; b.down_into_y = 1; b.filter = 0;
    b.mode = (d->p == 1 && d->q == 1 && skew == nullptr) ? BAND_PLAIN : BAND_GENERAL;
    b.skew = skew;

    const int64_t mbar = d->m / d->p, nbar = d->n / d->q, pq = (int64_t)d->p * d->q;
    const int64_t stages = plan.stages2d + plan.lead_total;
    // super-entries on the local anti-diagonal t of a slab, and the most that any slab holds at the global stage g
    auto on_stage = [&](int64_t t) -> int64_t {
        if (t < 0 || t >= plan.stages2d) return 0;
        const int64_t lo = t - nbar + 1 > 0 ? t - nbar + 1 : 0, hi = t + 1 < mbar ? t + 1 : mbar;
        return hi - lo;
    };
    // the reference's clamping rules (gptq_2d.py:1327-1329)
    const int64_t inner = d->inner_block > 0 && d->inner_block <= stages ? d->inner_block : stages;
    const int64_t outer = d->outer_block > inner && d->outer_block < stages ? d->outer_block : inner;
    const int T = d->p * d->q;
    for (int64_t outer_start = 0; outer_start < stages; outer_start += outer) {
        const int64_t outer_stop = outer_start + outer < stages ? outer_start + outer : stages;
        for (int64_t s0 = outer_start; s0 < outer_stop; s0 += inner) {
            const int64_t s1 = s0 + inner < outer_stop ? s0 + inner : outer_stop;
            for (int64_t s = s0; s < s1; ++s) {
                int64_t dmax = 0;
                for (int64_t behind = 0; behind <= plan.lead_total; ++behind) dmax = on_stage(s - behind) > dmax ? on_stage(s - behind) : dmax;
                if (dmax == 0) continue;
                A.stage = s; A.dmax = dmax;
                const int64_t work = d->batch * dmax * pq;
                if (d->lead_count > 0) {
                    fold_kernel<F><<<blocks_for(work, 128), 128, 0, st>>>(A);
                    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
                }
                switch (d->quant_kind) {
                case G2D_Q_ROUND: quantize_entries_kernel<F, G2D_Q_ROUND><<<blocks_for(work, 128), 128, 0, st>>>(A); break;
                case G2D_Q_AFFINE: quantize_entries_kernel<F, G2D_Q_AFFINE><<<blocks_for(work, 128), 128, 0, st>>>(A); break;
                case G2D_Q_ABSMAX_DYNAMIC: quantize_absmax_kernel<F><<<blocks_for(d->batch * dmax * d->p * 32, 128), 128, 0, st>>>(A); break;
                default: quantize_entries_kernel<F, G2D_Q_TRELLIS><<<blocks_for(work, 128), 128, 0, st>>>(A); break;
                }
                if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
                if (d->quant_kind == G2D_Q_TRELLIS) {
                    uint8_t *stage_codes = d->codes ? (uint8_t *)(ws + plan.stage_codes) : nullptr;
                    const TrellisIndex index{d->table_distinct, d->table_ids, d->table_distinct_count};
                    const int status = launch_trellis(d->dtype, d->batch * dmax, T, A.xs, d->table, d->trellis_L, d->trellis_K, d->trellis_V,
                                                      d->tail_biting, A.row_scale, z, nullptr, ws + plan.viterbi, stage_codes, st,
                                                      d->table_ids != nullptr ? &index : nullptr);
                    if (status != G2D_OK) return status;
                    if (stage_codes) {
                        scatter_codes_kernel<F><<<blocks_for(d->batch * dmax * plan.code_bytes, 256), 256, 0, st>>>(A, stage_codes, d->codes, plan.code_bytes);
                        if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
                    }
                }
                if (d->lead_count > 0) {
                    fold_commit_kernel<F><<<blocks_for(work, 128), 128, 0, st>>>(A);
                    if (check_launch() != G2D_OK) return G2D_ERR_CUDA;
                }
                const int status = launch_stage_push<F>(sd, z, s, s1, st, skew, dmax * pq);
                if (status != G2D_OK) return status;
            }
            if (s1 < outer_stop) {
                b.s0 = s0; b.s1 = s1; b.s_end = outer_stop;
                const int status = launch_band_update<F>(b, st);
                if (status != G2D_OK) return status;
            }
        }
        if (outer_stop < stages) {
            b.s0 = outer_start; b.s1 = outer_stop; b.s_end = stages;
            const int status = launch_band_update<F>(b, st);
            if (status != G2D_OK) return status;
        }
    }
    return G2D_OK;
}

}  // namespace

}  // namespace g2d

using namespace g2d;

extern "C" int g2d_super_workspace_bytes(const g2d_super_desc *desc, size_t *bytes) {
    const int status = check_super(desc);
    if (status != G2D_OK || !bytes) return status != G2D_OK ? status : G2D_ERR_BAD_ARGUMENT;
    Plan plan;
    make_plan(desc, &plan);
    *bytes = plan.total;
    return G2D_OK;
}

extern "C" int g2d_sweep_super_entry(const g2d_super_desc *desc, void *stream) {
    const int status = check_super(desc);
    if (status != G2D_OK) return status;
    if (desc->batch == 0 || desc->m == 0 || desc->n == 0) return G2D_OK;
    if (!desc->y || !desc->l || !desc->u) return G2D_ERR_BAD_ARGUMENT;
    if (desc->quant_kind == G2D_Q_AFFINE && (!desc->scale || !desc->zero)) return G2D_ERR_BAD_ARGUMENT;
    if (desc->quant_kind == G2D_Q_TRELLIS && (!desc->scale || !desc->table)) return G2D_ERR_BAD_ARGUMENT;
    if (desc->table_ids != nullptr && (!desc->table_distinct || desc->table_distinct_count <= 0 || ((uintptr_t)desc->table_ids & 15) != 0))
        return G2D_ERR_BAD_ARGUMENT;
    if (desc->quant_kind == G2D_Q_ABSMAX_DYNAMIC && desc->half != G2D_FP16 && desc->half != G2D_BF16) return G2D_ERR_BAD_ARGUMENT;
    for (int k = 0; k < desc->lead_count; ++k)
        if (!desc->lead_factor[k]) return G2D_ERR_BAD_ARGUMENT;
    if (desc->m / desc->p + desc->n / desc->q > (int64_t)1 << 30) return G2D_ERR_TOO_LARGE;
    Plan plan;
    make_plan(desc, &plan);
    if (!desc->workspace || desc->workspace_bytes < plan.total || ((uintptr_t)desc->workspace & 255) != 0) return G2D_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    return desc->dtype == G2D_F32 ? sweep_super<float>(desc, plan, st) : sweep_super<double>(desc, plan, st);
}
