// Packed integer codes of a rounded matrix, and back.
//
// The reference returns dequantised floats only and notes that the code can be recovered from them
// (quantizer_trellis.py:11-14; for the affine quantizer code = rint(z / scale + zero point), quantizer_int.py:63-83).
// A deployment stores the codes: here `bits`-bit unsigned fields code - qmin, packed little-endian (entry j of a row
// occupies the bits j * bits .. j * bits + bits - 1 of the row's byte string), every row padded to whole bytes.
// One thread handles eight consecutive entries of a row, i.e. `bits` whole bytes: 32 bytes in, `bits` bytes out.
// Pure streaming work, bound by HBM bandwidth: 4 (or 8) bytes read and bits / 8 bytes written per entry.
#include "g2d_common.cuh"

namespace g2d {

// Eight consecutive entries of a row of a matrix whose column stride is 0 (one value per row), 1 or anything else;
// entries past the row's end read as `fill`.  `vec` promises a unit column stride, eight whole entries and 16-byte alignment.
template <typename F>
__device__ __forceinline__ void load8(const F *__restrict__ row, int64_t c0, int64_t cs, int64_t n, bool vec, F fill, F (&v)[8]) {
    if (cs == 0) {
        const F one = row[0];
#pragma unroll
        for (int x = 0; x < 8; ++x) v[x] = one;
    } else if (vec && c0 + 8 <= n) {
        if constexpr (sizeof(F) == 4) {
            const float4 a = *reinterpret_cast<const float4 *>(row + c0), b = *reinterpret_cast<const float4 *>(row + c0 + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int x = 0; x < 8; x += 2) {
                const double2 a = *reinterpret_cast<const double2 *>(row + c0 + x);
                v[x] = a.x; v[x + 1] = a.y;
            }
        }
    } else {
#pragma unroll
        for (int x = 0; x < 8; ++x) v[x] = c0 + x < n ? row[(c0 + x) * cs] : fill;
    }
}

template <typename F>
__global__ void pack_codes_kernel(int64_t m, int64_t n, const F *__restrict__ z, const F *__restrict__ scale, int64_t srs, int64_t scs,
                                  const F *__restrict__ zero, int64_t zrs, int64_t zcs, F qmin, int bits, unsigned char *__restrict__ out,
                                  int64_t row_bytes) {
    const int64_t groups = ceil_div(n, (int64_t)8), total = m * groups;
    const unsigned top = (1u << bits) - 1u;
    const bool vec_z = n % 4 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0;
    const bool vec_s = scs == 1 && srs % 4 == 0 && reinterpret_cast<uintptr_t>(scale) % 16 == 0;
    const bool vec_o = zcs == 1 && zrs % 4 == 0 && reinterpret_cast<uintptr_t>(zero) % 16 == 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / groups, c0 = (t % groups) * 8;
        F zv[8], sv[8], ov[8];
        load8(z + r * n, c0, 1, n, vec_z, (F)0, zv);
        load8(scale + r * srs, c0, scs, n, vec_s, (F)1, sv);
        load8(zero + r * zrs, c0, zcs, n, vec_o, (F)0, ov);
        unsigned long long field = 0;  // 8 codes of at most 8 bits
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            if (c0 + x < n) {
                const F q = rint_even(add_rn(div_rn(zv[x], sv[x]), ov[x])) - qmin;
                const unsigned code = q < (F)0 ? 0u : (q > (F)top ? top : (unsigned)q);
                field |= (unsigned long long)code << (x * bits);
            }
        }
        unsigned char *dst = out + r * row_bytes + (c0 / 8) * bits;
        const int64_t left = row_bytes - (c0 / 8) * bits;  // a ragged last group owns fewer than `bits` bytes
        for (int b = 0; b < bits && b < left; ++b) dst[b] = (unsigned char)(field >> (8 * b));
    }
}

template <typename F>
__global__ void unpack_codes_kernel(int64_t m, int64_t n, const unsigned char *__restrict__ codes, int64_t row_bytes,
                                    const F *__restrict__ scale, int64_t srs, int64_t scs, const F *__restrict__ zero, int64_t zrs,
                                    int64_t zcs, F qmin, int bits, F *__restrict__ z) {
    const int64_t groups = ceil_div(n, (int64_t)8), total = m * groups;
    const unsigned top = (1u << bits) - 1u;
    const bool vec_z = n % 4 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0;
    const bool vec_s = scs == 1 && srs % 4 == 0 && reinterpret_cast<uintptr_t>(scale) % 16 == 0;
    const bool vec_o = zcs == 1 && zrs % 4 == 0 && reinterpret_cast<uintptr_t>(zero) % 16 == 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / groups, c0 = (t % groups) * 8;
        const unsigned char *src = codes + r * row_bytes + (c0 / 8) * bits;
        const int64_t left = row_bytes - (c0 / 8) * bits;
        unsigned long long field = 0;
        for (int b = 0; b < bits && b < left; ++b) field |= (unsigned long long)src[b] << (8 * b);
        F sv[8], ov[8], zv[8];
        load8(scale + r * srs, c0, scs, n, vec_s, (F)1, sv);
        load8(zero + r * zrs, c0, zcs, n, vec_o, (F)0, ov);
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const F q = (F)((unsigned)(field >> (x * bits)) & top) + qmin;
            zv[x] = mul_rn(sub_rn(q, ov[x]), sv[x]);  // as the affine quantizer forms its value
        }
        if (vec_z && c0 + 8 <= n && sizeof(F) == 4) {
            float4 *dst = reinterpret_cast<float4 *>(z + r * n + c0);
            dst[0] = make_float4((float)zv[0], (float)zv[1], (float)zv[2], (float)zv[3]);
            dst[1] = make_float4((float)zv[4], (float)zv[5], (float)zv[6], (float)zv[7]);
        } else {
#pragma unroll
            for (int x = 0; x < 8; ++x)
                if (c0 + x < n) z[r * n + c0 + x] = zv[x];
        }
    }
}

static unsigned pack_grid(int64_t m, int64_t n) {
    const int64_t blocks = ceil_div(m * ceil_div(n, (int64_t)8), (int64_t)256);
    return (unsigned)(blocks < 148 * 32 ? (blocks > 0 ? blocks : 1) : 148 * 32);
}

}  // namespace g2d

using namespace g2d;

static int pack_check(int dtype, int64_t m, int64_t n, const void *a, const void *scale, const void *zero, int bits, const void *b, int64_t row_bytes) {
    if ((dtype != G2D_F32 && dtype != G2D_F64) || m < 0 || n < 0 || bits < 1 || bits > 8) return G2D_ERR_BAD_ARGUMENT;
    if (m == 0 || n == 0) return G2D_OK;
    if (!a || !scale || !zero || !b || row_bytes < (n * bits + 7) / 8) return G2D_ERR_BAD_ARGUMENT;
    return G2D_OK;
}

extern "C" int g2d_pack_codes(int dtype, int64_t m, int64_t n, const void *z, const void *scale, int64_t scale_row_stride,
                              int64_t scale_col_stride, const void *zero, int64_t zero_row_stride, int64_t zero_col_stride, double qmin,
                              int32_t bits, uint8_t *codes, int64_t row_bytes, void *stream) {
    const int status = pack_check(dtype, m, n, z, scale, zero, bits, codes, row_bytes);
    if (status != G2D_OK || m == 0 || n == 0) return status;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32)
        pack_codes_kernel<float><<<pack_grid(m, n), 256, 0, st>>>(m, n, (const float *)z, (const float *)scale, scale_row_stride, scale_col_stride,
                                                                 (const float *)zero, zero_row_stride, zero_col_stride, (float)qmin, bits, codes, row_bytes);
    else
        pack_codes_kernel<double><<<pack_grid(m, n), 256, 0, st>>>(m, n, (const double *)z, (const double *)scale, scale_row_stride, scale_col_stride,
                                                                  (const double *)zero, zero_row_stride, zero_col_stride, qmin, bits, codes, row_bytes);
    return check_launch();
}

extern "C" int g2d_unpack_codes(int dtype, int64_t m, int64_t n, const uint8_t *codes, int64_t row_bytes, const void *scale,
                                int64_t scale_row_stride, int64_t scale_col_stride, const void *zero, int64_t zero_row_stride,
                                int64_t zero_col_stride, double qmin, int32_t bits, void *z, void *stream) {
    const int status = pack_check(dtype, m, n, z, scale, zero, bits, codes, row_bytes);
    if (status != G2D_OK || m == 0 || n == 0) return status;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32)
        unpack_codes_kernel<float><<<pack_grid(m, n), 256, 0, st>>>(m, n, codes, row_bytes, (const float *)scale, scale_row_stride, scale_col_stride,
                                                                   (const float *)zero, zero_row_stride, zero_col_stride, (float)qmin, bits, (float *)z);
    else
        unpack_codes_kernel<double><<<pack_grid(m, n), 256, 0, st>>>(m, n, codes, row_bytes, (const double *)scale, scale_row_stride, scale_col_stride,
                                                                    (const double *)zero, zero_row_stride, zero_col_stride, qmin, bits, (double *)z);
    return check_launch();
}
