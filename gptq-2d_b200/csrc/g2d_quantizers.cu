// INT quantizer kernels: strided / super-entry affine quantize-dequantize, row abs-max scales and the
// dynamic abs-max quantizer.  They replace the four Triton kernels of the reference's quantizer_int.py
// (:160, :247, :366, :407) bit for bit: IEEE division, round half to even, denormals kept, the scale
// rounded to fp16 / bf16 through fp32.
#include "g2d_common.cuh"

namespace g2d {

template <typename F>
__global__ void affine_strided_kernel(int64_t batch, int64_t matrix_size, int64_t start, int64_t step, int64_t count,
                                      const F *__restrict__ y, const F *__restrict__ scale, const int64_t *scale_off,
                                      const F *__restrict__ zero, const int64_t *zero_off, F qmin, F qmax, F *__restrict__ out) {
    const int64_t total = batch * count;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / count, k = t % count;
        const int64_t pos = start + k * step;
        const F s = scale[(scale_off ? scale_off[b] : 0) + pos], z = zero[(zero_off ? zero_off[b] : 0) + pos];
        out[t] = affine_value(y[b * matrix_size + pos], s, z, qmin, qmax);
    }
}

template <typename F>
__global__ void affine_super_entry_kernel(int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int p, int q,
                                          int64_t stride_d, int64_t stride_p, int64_t stride_q, const F *__restrict__ y,
                                          const F *__restrict__ scale, const int64_t *scale_off, const F *__restrict__ zero,
                                          const int64_t *zero_off, F qmin, F qmax, F *__restrict__ out) {
    const int64_t per = d * p * q, total = batch * per;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / per, e = t % per;
        const int64_t k = e / ((int64_t)p * q), r = e / q % p, c = e % q;
        const int64_t pos = first + k * stride_d + r * stride_p + c * stride_q;
        const F s = scale[(scale_off ? scale_off[b] : 0) + pos], z = zero[(zero_off ? zero_off[b] : 0) + pos];
        out[t] = affine_value(y[b * matrix_size + pos], s, z, qmin, qmax);
    }
}

// one warp per row
template <typename F>
__global__ void absmax_scale_kernel(int64_t rows, int64_t size, int64_t row_stride, int64_t col_stride, const F *__restrict__ x,
                                    F divisor, int half_kind, F *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        F a = (F)0;
        for (int64_t c = lane; c < size; c += 32) a = fmax(a, fabs(x[row * row_stride + c * col_stride]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmax(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) out[row] = absmax_scale_value(a, divisor, half_kind);
    }
}

// one warp per row of a selected super-entry: row index = (batch, k, r)
template <typename F>
__global__ void absmax_quantize_kernel(int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int p, int q,
                                       int64_t stride_d, int64_t stride_p, int64_t stride_q, const F *__restrict__ y,
                                       F qmin, F qmax, F divisor, int half_kind, F *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5, rows = batch * d * p;
    for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const int64_t b = row / (d * p), k = row / p % d, r = row % p;
        const F *src = y + b * matrix_size + first + k * stride_d + r * stride_p;
        F a = (F)0;
        for (int64_t c = lane; c < q; c += 32) a = fmax(a, fabs(src[c * stride_q]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmax(a, __shfl_xor_sync(0xffffffffu, a, o));
        const F s = absmax_scale_value(a, divisor, half_kind);
        for (int64_t c = lane; c < q; c += 32) {
            F t = rint_even(div_rn(src[c * stride_q], s));
            t = t < qmin ? qmin : t;
            t = t > qmax ? qmax : t;
            out[row * q + c] = mul_rn(t, s);
        }
    }
}

static inline unsigned grid_for(int64_t work, int threads) {
    int64_t blocks = ceil_div(work, threads);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 32) blocks = 148 * 32;
    return (unsigned)blocks;
}

template <typename F>
static int affine_strided(int64_t batch, int64_t matrix_size, int64_t start, int64_t step, int64_t count, const void *y,
                          const void *scale, const int64_t *so, const void *zero, const int64_t *zo, double qmin, double qmax,
                          void *out, cudaStream_t st) {
    affine_strided_kernel<F><<<grid_for(batch * count, 256), 256, 0, st>>>(batch, matrix_size, start, step, count, (const F *)y,
                                                                         (const F *)scale, so, (const F *)zero, zo, (F)qmin, (F)qmax, (F *)out);
    return check_launch();
}

template <typename F>
static int affine_se(int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int p, int q, int64_t sd, int64_t sp, int64_t sq,
                     const void *y, const void *scale, const int64_t *so, const void *zero, const int64_t *zo, double qmin,
                     double qmax, void *out, cudaStream_t st) {
    affine_super_entry_kernel<F><<<grid_for(batch * d * p * q, 256), 256, 0, st>>>(
        batch, matrix_size, first, d, p, q, sd, sp, sq, (const F *)y, (const F *)scale, so, (const F *)zero, zo, (F)qmin, (F)qmax, (F *)out);
    return check_launch();
}

}  // namespace g2d

using namespace g2d;

extern "C" int g2d_affine_quantize(int dtype, int64_t batch, int64_t matrix_size, int64_t start, int64_t step, int64_t count,
                                   const void *y, const void *scale, const int64_t *scale_offsets, const void *zero,
                                   const int64_t *zero_offsets, double qmin, double qmax, void *out, void *stream) {
    if (batch < 0 || count < 0 || step <= 0 || start < 0 || !(qmin < qmax)) return G2D_ERR_BAD_ARGUMENT;
    if (batch == 0 || count == 0) return G2D_OK;
    if (!y || !scale || !zero || !out) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32) return affine_strided<float>(batch, matrix_size, start, step, count, y, scale, scale_offsets, zero, zero_offsets, qmin, qmax, out, st);
    if (dtype == G2D_F64) return affine_strided<double>(batch, matrix_size, start, step, count, y, scale, scale_offsets, zero, zero_offsets, qmin, qmax, out, st);
    return G2D_ERR_BAD_ARGUMENT;
}

extern "C" int g2d_affine_quantize_super_entry(int dtype, int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int32_t p,
                                               int32_t q, int64_t stride_d, int64_t stride_p, int64_t stride_q, const void *y,
                                               const void *scale, const int64_t *scale_offsets, const void *zero,
                                               const int64_t *zero_offsets, double qmin, double qmax, void *out, void *stream) {
    if (batch < 0 || d < 0 || p <= 0 || q <= 0 || first < 0 || !(qmin < qmax)) return G2D_ERR_BAD_ARGUMENT;
    if (batch == 0 || d == 0) return G2D_OK;
    if (!y || !scale || !zero || !out) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32) return affine_se<float>(batch, matrix_size, first, d, p, q, stride_d, stride_p, stride_q, y, scale, scale_offsets, zero, zero_offsets, qmin, qmax, out, st);
    if (dtype == G2D_F64) return affine_se<double>(batch, matrix_size, first, d, p, q, stride_d, stride_p, stride_q, y, scale, scale_offsets, zero, zero_offsets, qmin, qmax, out, st);
    return G2D_ERR_BAD_ARGUMENT;
}

extern "C" int g2d_absmax_scale(int dtype, int64_t rows, int64_t size, int64_t row_stride, int64_t col_stride, const void *x,
                                double qmin, double qmax, int half, void *out, void *stream) {
    if (rows < 0 || size < 0 || !(qmin < qmax) || (half != G2D_FP16 && half != G2D_BF16)) return G2D_ERR_BAD_ARGUMENT;
    if (rows == 0) return G2D_OK;
    if (!x || !out) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    const double divisor = (qmax - qmin) / 2.0;
    if (dtype == G2D_F32)
        absmax_scale_kernel<float><<<grid_for(rows * 32, 256), 256, 0, st>>>(rows, size, row_stride, col_stride, (const float *)x, (float)divisor, half, (float *)out);
    else if (dtype == G2D_F64)
        absmax_scale_kernel<double><<<grid_for(rows * 32, 256), 256, 0, st>>>(rows, size, row_stride, col_stride, (const double *)x, divisor, half, (double *)out);
    else
        return G2D_ERR_BAD_ARGUMENT;
    return check_launch();
}

extern "C" int g2d_absmax_quantize_super_entry(int dtype, int64_t batch, int64_t matrix_size, int64_t first, int64_t d, int32_t p,
                                               int32_t q, int64_t stride_d, int64_t stride_p, int64_t stride_q, const void *y,
                                               double qmin, double qmax, int half, void *out, void *stream) {
    if (batch < 0 || d < 0 || p <= 0 || q <= 0 || first < 0 || !(qmin < qmax) || (half != G2D_FP16 && half != G2D_BF16))
        return G2D_ERR_BAD_ARGUMENT;
    if (batch == 0 || d == 0) return G2D_OK;
    if (!y || !out) return G2D_ERR_BAD_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    const double divisor = (qmax - qmin) / 2.0;
    const int64_t rows = batch * d * p;
    if (dtype == G2D_F32)
        absmax_quantize_kernel<float><<<grid_for(rows * 32, 128), 128, 0, st>>>(batch, matrix_size, first, d, p, q, stride_d, stride_p, stride_q,
                                                                                (const float *)y, (float)qmin, (float)qmax, (float)divisor, half, (float *)out);
    else if (dtype == G2D_F64)
        absmax_quantize_kernel<double><<<grid_for(rows * 32, 128), 128, 0, st>>>(batch, matrix_size, first, d, p, q, stride_d, stride_p, stride_q,
                                                                                 (const double *)y, qmin, qmax, divisor, half, (double *)out);
    else
        return G2D_ERR_BAD_ARGUMENT;
    return check_launch();
}
