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
// entries past the row's end read as `fill`.  `vec` promises a unit column stride and 32-byte alignment of every group of eight.
template <typename F>
__device__ __forceinline__ void load8(const F *__restrict__ row, int64_t c0, int64_t cs, int64_t n, bool vec, F fill, F (&v)[8]) {
    if (cs == 0) {
        const F one = row[0];
#pragma unroll
        for (int x = 0; x < 8; ++x) v[x] = one;
    } else if (vec && c0 + 8 <= n) {
        if constexpr (sizeof(F) == 4) {
            // one 32-byte load: consecutive lanes then cover whole sectors with every instruction
            asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                         : "l"(row + c0));
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

// z / s for the code of a value on the quantizer's grid.  float: the product with the correctly rounded reciprocal
// plus one residual correction, which is the IEEE quotient except, rarely, in its last bit; a rounded value lies
// within an ulp of (code - zero point) * scale, so its code never depends on that bit.  double: IEEE division.
__device__ __forceinline__ float reciprocal(float s) { return __frcp_rn(s); }
__device__ __forceinline__ double reciprocal(double) { return 0.0; }
__device__ __forceinline__ float quotient(float z, float s, float rc) {
    const float q0 = z * rc;
    const float q1 = fmaf(fmaf(-q0, s, z), rc, q0);
    return (fabsf(s) > 1e-30f && fabsf(s) < 1e30f && fabsf(q1) < 1e30f) ? q1 : div_rn(z, s);  // extreme scales take the exact path
}
__device__ __forceinline__ double quotient(double z, double s, double) { return div_rn(z, s); }
__device__ __forceinline__ int to_int_rn(float a) { return __float2int_rn(a); }
__device__ __forceinline__ int to_int_rn(double a) { return __double2int_rn(a); }

template <typename F, int BITS>
__global__ void __launch_bounds__(256, 3) pack_codes_kernel(int64_t m, int64_t n, const F *__restrict__ z, const F *__restrict__ scale, int64_t srs,
                                                            int64_t scs, const F *__restrict__ zero, int64_t zrs, int64_t zcs, F qmin,
                                                            unsigned char *__restrict__ out, int64_t row_bytes) {
    constexpr int bits = BITS;  // the field width as a compile-time constant: shifts and store widths are immediates
    // a thread takes two neighbouring groups of eight entries; all its loads are issued before any arithmetic
    const int64_t groups = ceil_div(n, (int64_t)8), pairs = ceil_div(groups, (int64_t)2), total = m * pairs;
    const unsigned top = (1u << bits) - 1u;
    const int qmin_int = to_int_rn(qmin);  // an integer by contract
    const bool vec_z = n % 8 == 0 && reinterpret_cast<uintptr_t>(z) % 32 == 0;
    const bool vec_s = scs == 1 && srs % 8 == 0 && reinterpret_cast<uintptr_t>(scale) % 32 == 0;
    const bool vec_o = zcs == 1 && zrs % 8 == 0 && reinterpret_cast<uintptr_t>(zero) % 32 == 0;
    const bool wide = (bits == 2 || bits == 4 || bits == 8) && row_bytes % bits == 0 && reinterpret_cast<uintptr_t>(out) % bits == 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / pairs, g0 = (t % pairs) * 2;
        F zv[2][8], sv[2][8], ov[2][8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t c0 = (g0 + h) * 8;
            load8(z + r * n, c0, 1, n, vec_z, (F)0, zv[h]);
            load8(scale + r * srs, c0, scs, n, vec_s, (F)1, sv[h]);
            load8(zero + r * zrs, c0, zcs, n, vec_o, (F)0, ov[h]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t c0 = (g0 + h) * 8;
            if (c0 >= n) continue;
            const F row_rc = reciprocal(sv[h][0]);  // shared by the group when the scale is per row
            unsigned half_field[2] = {0u, 0u};      // four codes of at most 8 bits each
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                if (c0 + x < n) {
                    const F rc = scs == 0 ? row_rc : reciprocal(sv[h][x]);
                    // round half to even and convert in one step (the conversion saturates); the clamp is done on
                    // integers: the field's bounds moved by qmin, both well inside the int range
                    int q = to_int_rn(add_rn(quotient(zv[h][x], sv[h][x], rc), ov[h][x]));
                    q = q < qmin_int ? qmin_int : (q > qmin_int + (int)top ? qmin_int + (int)top : q);
                    half_field[x >> 2] |= (unsigned)(q - qmin_int) << ((x & 3) * bits);
                }
            }
            const unsigned long long field = (unsigned long long)half_field[0] | ((unsigned long long)half_field[1] << (4 * bits));
            unsigned char *dst = out + r * row_bytes + (c0 / 8) * bits;
            const int64_t left = row_bytes - (c0 / 8) * bits;  // a ragged last group owns fewer than `bits` bytes
            if (wide && left >= bits) {  // the group's bytes as one aligned word
                if (bits == 4) *reinterpret_cast<unsigned *>(dst) = (unsigned)field;
                else if (bits == 8) *reinterpret_cast<unsigned long long *>(dst) = field;
                else *reinterpret_cast<unsigned short *>(dst) = (unsigned short)field;
            } else {
                for (int b = 0; b < bits && b < left; ++b) dst[b] = (unsigned char)(field >> (8 * b));
            }
        }
    }
}

template <typename F>
__global__ void unpack_codes_kernel(int64_t m, int64_t n, const unsigned char *__restrict__ codes, int64_t row_bytes,
                                    const F *__restrict__ scale, int64_t srs, int64_t scs, const F *__restrict__ zero, int64_t zrs,
                                    int64_t zcs, F qmin, int bits, F *__restrict__ z) {
    const int64_t groups = ceil_div(n, (int64_t)8), total = m * groups;
    const unsigned top = (1u << bits) - 1u;
    const bool vec_z = n % 8 == 0 && reinterpret_cast<uintptr_t>(z) % 32 == 0;
    const bool vec_s = scs == 1 && srs % 8 == 0 && reinterpret_cast<uintptr_t>(scale) % 32 == 0;
    const bool vec_o = zcs == 1 && zrs % 8 == 0 && reinterpret_cast<uintptr_t>(zero) % 32 == 0;
    const bool wide = (bits == 2 || bits == 4 || bits == 8) && row_bytes % bits == 0 && reinterpret_cast<uintptr_t>(codes) % bits == 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / groups, c0 = (t % groups) * 8;
        const unsigned char *src = codes + r * row_bytes + (c0 / 8) * bits;
        const int64_t left = row_bytes - (c0 / 8) * bits;
        unsigned long long field = 0;
        if (wide && left >= bits) {
            if (bits == 4) field = *reinterpret_cast<const unsigned *>(src);
            else if (bits == 8) field = *reinterpret_cast<const unsigned long long *>(src);
            else field = *reinterpret_cast<const unsigned short *>(src);
        } else {
            for (int b = 0; b < bits && b < left; ++b) field |= (unsigned long long)src[b] << (8 * b);
        }
        F sv[8], ov[8], zv[8];
        load8(scale + r * srs, c0, scs, n, vec_s, (F)1, sv);
        load8(zero + r * zrs, c0, zcs, n, vec_o, (F)0, ov);
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const F q = (F)((unsigned)(field >> (x * bits)) & top) + qmin;
            zv[x] = mul_rn(sub_rn(q, ov[x]), sv[x]);  // as the affine quantizer forms its value
        }
        if (vec_z && c0 + 8 <= n && sizeof(F) == 4) {
            asm volatile("st.global.v8.f32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::"f"((float)zv[0]), "f"((float)zv[1]), "f"((float)zv[2]),
                         "f"((float)zv[3]), "f"((float)zv[4]), "f"((float)zv[5]), "f"((float)zv[6]), "f"((float)zv[7]), "l"(z + r * n + c0)
                         : "memory");
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

// Full symmetric matrix from its packed lower triangle: one CTA per 32 x 32 tile on or below the diagonal reads its rows
// of the packed array (row i starts at i (i + 1) / 2) and writes the tile and, through shared memory, its mirror image.
template <typename F>
__global__ void symmetric_from_packed_kernel(int64_t n, const F *__restrict__ packed, F *__restrict__ out) {
    __shared__ F tile[32][33];
    const int64_t tiles = ceil_div(n, (int64_t)32), count = tiles * (tiles + 1) / 2;
    for (int64_t t = blockIdx.x; t < count; t += gridDim.x) {
        int64_t bi = (int64_t)((sqrt(8.0 * (double)t + 1.0) - 1.0) / 2.0);
        while ((bi + 1) * (bi + 2) / 2 <= t) ++bi;
        while (bi * (bi + 1) / 2 > t) --bi;
        const int64_t bj = t - bi * (bi + 1) / 2;
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t i = bi * 32 + r, j = bj * 32 + threadIdx.x;
            F v = (F)0;
            if (i < n && j <= i) {
                v = packed[i * (i + 1) / 2 + j];
                out[i * n + j] = v;
            }
            tile[r][threadIdx.x] = v;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const int64_t j = bj * 32 + r, i = bi * 32 + threadIdx.x;  // the mirrored entry (j, i), j < i
            if (i < n && j < i) out[j * n + i] = tile[threadIdx.x][r];
        }
        __syncthreads();
    }
}

}  // namespace g2d

using namespace g2d;

extern "C" int g2d_symmetric_from_packed(int dtype, int64_t n, const void *packed, void *out, void *stream) {
    if ((dtype != G2D_F32 && dtype != G2D_F64) || n < 0) return G2D_ERR_BAD_ARGUMENT;
    if (n == 0) return G2D_OK;
    if (!packed || !out) return G2D_ERR_BAD_ARGUMENT;
    const int64_t tiles = ceil_div(n, (int64_t)32), count = tiles * (tiles + 1) / 2;
    const unsigned grid = (unsigned)(count < 148 * 16 ? count : 148 * 16);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32) symmetric_from_packed_kernel<float><<<grid, dim3(32, 8), 0, st>>>(n, (const float *)packed, (float *)out);
    else symmetric_from_packed_kernel<double><<<grid, dim3(32, 8), 0, st>>>(n, (const double *)packed, (double *)out);
    return check_launch();
}

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
    const unsigned grid = pack_grid(m, n);
#define G2D_PACK_CASE(B)                                                                                                                     \
    case B:                                                                                                                                  \
        if (dtype == G2D_F32)                                                                                                                \
            pack_codes_kernel<float, B><<<grid, 256, 0, st>>>(m, n, (const float *)z, (const float *)scale, scale_row_stride, scale_col_stride, \
                                                              (const float *)zero, zero_row_stride, zero_col_stride, (float)qmin, codes, row_bytes); \
        else                                                                                                                                 \
            pack_codes_kernel<double, B><<<grid, 256, 0, st>>>(m, n, (const double *)z, (const double *)scale, scale_row_stride, scale_col_stride, \
                                                               (const double *)zero, zero_row_stride, zero_col_stride, qmin, codes, row_bytes); \
        break;
    switch (bits) {
        G2D_PACK_CASE(1) G2D_PACK_CASE(2) G2D_PACK_CASE(3) G2D_PACK_CASE(4) G2D_PACK_CASE(5) G2D_PACK_CASE(6) G2D_PACK_CASE(7) G2D_PACK_CASE(8)
    default: return G2D_ERR_BAD_ARGUMENT;
    }
#undef G2D_PACK_CASE
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
