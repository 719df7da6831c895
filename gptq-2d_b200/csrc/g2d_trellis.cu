// Bitshift-trellis (QTIP) quantizer: Viterbi search as a shared-memory dynamic program.
//
// Replaces _viterbi_step_kernel / _viterbi_final_kernel / _viterbi_backtrack_kernel of the reference
// (quantizer_trellis.py:146-268) and reproduces _trellis_quantize_torch (:121-143) bit for bit: costs are
// (table - x)^2 summed over the V <= 2 values without fused multiply-adds, the running cost is added last,
// and every minimum takes the first index among equals.
//
// A state is an L-bit window; a step shifts in KV = K*V bits, so state s has the predecessors
// h * G + (s >> KV), h < 2^KV, G = 2^(L-KV).  All 2^KV states that share (s >> KV)... equivalently, the cost of a
// state is the minimum over its group of predecessors plus its own local cost, so only the G group minima
// of every step are kept:  B_t[g] = min_h (B_{t-1}[(h G + g) >> KV] + local_t[h G + g]).
// One CTA runs R sequences at once: B_t and B_{t-1} of each live in shared memory (2 R G values), every
// table entry is loaded once per step for all R sequences, and one barrier separates the steps.  The
// arg-min h of every (step, group) goes to global scratch (one byte each) for the walk back.
//
// Packed paths.  A path is also emitted as its bit string, the storage format of a trellis code (T K bits per sequence
// when tail-biting; the reference only notes that "the T K-bit code can be recovered", quantizer_trellis.py:11-14).
// The string is the sequence of the K V bits that every step shifts into the state, most significant bit first,
// preceded, when the path is not tail-biting, by the L - K V upper bits of the first state (tail-biting paths need no
// header: their first state continues the end of the string).  State t is then the L bits of the string that end
// with step t's symbol, read circularly for a tail-biting path.  Bit i of the string is bit i % 8 of byte i / 8.
#include "g2d_common.cuh"

namespace g2d {

constexpr int VT = 512;  // threads per CTA

template <typename F>
__device__ __forceinline__ F local_cost(const F *__restrict__ table, int64_t s, int V, F x0, F x1) {
    const F d0 = sub_rn(table[s * V], x0);
    F c = mul_rn(d0, d0);
    if (V == 2) {
        const F d1 = sub_rn(table[s * V + 1], x1);
        c = add_rn(c, mul_rn(d1, d1));
    }
    return c;
}

template <typename F>
__device__ __forceinline__ F pos_inf() { return (F)INFINITY; }

// the two values of a table entry in one load (V = 2: entries are pairs, naturally aligned)
__device__ __forceinline__ void load_pair(const float *p, float &a, float &b) {
    const float2 t = *reinterpret_cast<const float2 *>(p);
    a = t.x; b = t.y;
}
__device__ __forceinline__ void load_pair(const double *p, double &a, double &b) {
    const double2 t = *reinterpret_cast<const double2 *>(p);
    a = t.x; b = t.y;
}

template <typename F, int R>
__global__ void __launch_bounds__(VT) viterbi_kernel(int64_t rows, int T, const F *__restrict__ x, const F *__restrict__ table,
                                                     int Lbits, int shift, int V, int tail_biting, const F *__restrict__ scale,
                                                     F *__restrict__ out, int64_t *__restrict__ states, uint8_t *__restrict__ choices,
                                                     uint8_t *__restrict__ codes, int64_t code_bytes) {
    extern __shared__ __align__(16) unsigned char g2d_vsmem[];
    const int64_t S = (int64_t)1 << Lbits, G = S >> shift;
    const int H = 1 << shift;
    const int steps = T / V;
    F *B = reinterpret_cast<F *>(g2d_vsmem);  // [2][R][G]
    __shared__ F red_val[VT / 32][R];
    __shared__ long long red_arg[VT / 32][R];
    __shared__ long long seq_state[R];    // state at the step the walk back starts from / stops at
    __shared__ long long seq_overlap[R];  // tail-biting overlap bits, -1 when unconstrained
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t slots = steps > 1 ? steps - 1 : 1;

    for (int64_t row0 = (int64_t)blockIdx.x * R; row0 < rows; row0 += (int64_t)gridDim.x * R) {
        if (tid < R) seq_overlap[tid] = -1;
        __syncthreads();
        for (int pass = tail_biting ? 0 : 1; pass < 2; ++pass) {
            const int half = steps / 2;
            const int roll = pass == 0 ? steps - half : 0;
            const int stop = pass == 0 ? half : 0;
            // ---- forward: group minima of the steps 0 .. steps-2 ----
            for (int t = 0; t + 1 < steps; ++t) {
                const F *prev = B + (size_t)((t + 1) & 1) * R * G;
                F *next = B + (size_t)(t & 1) * R * G;
                F x0[R], x1[R];
                long long ov[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int64_t row = row0 + r < rows ? row0 + r : rows - 1;
                    const F *xt = x + row * T + (int64_t)((t + roll) % steps) * V;
                    x0[r] = xt[0];
                    x1[r] = V == 2 ? xt[1] : (F)0;
                    ov[r] = seq_overlap[r];
                }
                const int Gi = (int)G;  // the states fit 32-bit arithmetic (L <= 24)
                int ovi[R];
#pragma unroll
                for (int r = 0; r < R; ++r) ovi[r] = (int)ov[r];
                // The common shape (sixteen predecessors, pairs of values, not the first step) has a path of its own:
                // everything that the generic loop below derives per predecessor is a constant stride here.
                const bool fast = H == 16 && V == 2 && t > 0 && (Gi & 15) == 0;
                for (int g = tid; fast && g < Gi; g += VT) {
                    const F *entry = table + 2 * g;            // predecessor h: + h * 2 Gi
                    const F *before = prev + (g >> 4);         // its group minimum: + h * (Gi >> 4), + r * Gi
                    const int table_stride = 2 * Gi, low_stride = Gi >> 4;
                    F best[R];
                    int arg[R];
#pragma unroll
                    for (int half_h = 0; half_h < 2; ++half_h) {
                        F tt0[8], tt1[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) load_pair(entry + (half_h * 8 + q) * table_stride, tt0[q], tt1[q]);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const int h = half_h * 8 + q;
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                const F d0 = sub_rn(tt0[q], x0[r]), d1 = sub_rn(tt1[q], x1[r]);
                                const F c = add_rn(before[r * Gi + h * low_stride], add_rn(mul_rn(d0, d0), mul_rn(d1, d1)));
                                if (h == 0 || c < best[r]) { best[r] = c; arg[r] = h; }
                            }
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        next[r * Gi + g] = best[r];
                        if (row0 + r < rows) choices[((row0 + r) * slots + t) * G + g] = (uint8_t)arg[r];
                    }
                }
                for (int g = tid; !fast && g < Gi; g += VT) {
                    F best[R];
                    int arg[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) { best[r] = pos_inf<F>(); arg[r] = 0; }
                    // the table entries of eight predecessors are fetched before any of them is used: a thread's loads
                    // (L2 hits: the table is larger than L1) overlap instead of queueing behind the running minimum
                    constexpr int HB = 8;
                    for (int h0 = 0; h0 < H; h0 += HB) {
                        F tt0[HB], tt1[HB];
#pragma unroll
                        for (int q = 0; q < HB; ++q) {
                            const int s = (h0 + q < H ? h0 + q : H - 1) * Gi + g;
                            if (V == 2) {
                                load_pair(table + 2 * s, tt0[q], tt1[q]);
                            } else {
                                tt0[q] = table[s];
                                tt1[q] = (F)0;
                            }
                        }
#pragma unroll
                        for (int q = 0; q < HB; ++q) {
                            const int h = h0 + q;
                            if (h >= H) break;
                            const int low = (h * Gi + g) >> shift;
                            const F t0 = tt0[q], t1 = tt1[q];
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                const F d0 = sub_rn(t0, x0[r]);
                                F c = mul_rn(d0, d0);
                                if (V == 2) {
                                    const F d1 = sub_rn(t1, x1[r]);
                                    c = add_rn(c, mul_rn(d1, d1));
                                }
                                if (t == 0) {
                                    if (ovi[r] >= 0 && low != ovi[r]) c = pos_inf<F>();
                                } else {
                                    c = add_rn(prev[r * Gi + low], c);
                                }
                                if (h == 0 || c < best[r]) { best[r] = c; arg[r] = h; }
                            }
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        next[(size_t)r * G + g] = best[r];
                        if (row0 + r < rows) choices[((row0 + r) * slots + t) * G + g] = (uint8_t)arg[r];
                    }
                }
                __syncthreads();
            }
            // ---- last step: first arg-min over all states, with the final mask ----
            {
                const int t = steps - 1;
                const F *prev = B + (size_t)((t + 1) & 1) * R * G;
                F best[R];
                long long arg[R];
#pragma unroll
                for (int r = 0; r < R; ++r) { best[r] = pos_inf<F>(); arg[r] = S; }
                F x0[R], x1[R];
                long long ov[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int64_t row = row0 + r < rows ? row0 + r : rows - 1;
                    const F *xt = x + row * T + (int64_t)((t + roll) % steps) * V;
                    x0[r] = xt[0];
                    x1[r] = V == 2 ? xt[1] : (F)0;
                    ov[r] = seq_overlap[r];
                }
                for (int64_t s = tid; s < S; s += VT) {
                    const F t0 = table[s * V], t1 = V == 2 ? table[s * V + 1] : (F)0;
                    const int64_t low = s >> shift;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const F d0 = sub_rn(t0, x0[r]);
                        F c = mul_rn(d0, d0);
                        if (V == 2) {
                            const F d1 = sub_rn(t1, x1[r]);
                            c = add_rn(c, mul_rn(d1, d1));
                        }
                        if (t == 0) {
                            if (ov[r] >= 0 && low != ov[r]) c = pos_inf<F>();
                        } else {
                            c = add_rn(prev[(size_t)r * G + low], c);
                        }
                        if (ov[r] >= 0 && (s & (G - 1)) != ov[r]) c = pos_inf<F>();
                        // ascending s within a thread: strict < keeps the first minimum
                        if (arg[r] == S || c < best[r]) { best[r] = c; arg[r] = s; }
                    }
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    F b = best[r];
                    long long a = arg[r];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const F ob = __shfl_xor_sync(0xffffffffu, b, o);
                        const long long oa = __shfl_xor_sync(0xffffffffu, a, o);
                        if (oa < S && (a >= S || ob < b || (ob == b && oa < a))) { b = ob; a = oa; }
                    }
                    if (lane == 0) { red_val[warp][r] = b; red_arg[warp][r] = a; }
                }
                __syncthreads();
                if (tid < R) {
                    F b = red_val[0][tid];
                    long long a = red_arg[0][tid];
                    for (int w = 1; w < VT / 32; ++w) {
                        const F ob = red_val[w][tid];
                        const long long oa = red_arg[w][tid];
                        if (oa < S && (a >= S || ob < b || (ob == b && oa < a))) { b = ob; a = oa; }
                    }
                    seq_state[tid] = a;
                }
                __syncthreads();
            }
            // ---- walk back: thread r follows sequence r ----
            if (tid < R && row0 + tid < rows) {
                const int64_t row = row0 + tid;
                long long state = seq_state[tid];
                const F sc = scale ? scale[row] : (F)1;
                uint8_t *code = (pass == 1 && codes) ? codes + row * code_bytes : nullptr;
                const int header = tail_biting ? 0 : Lbits - shift;
                if (code)
                    for (int64_t b = 0; b < code_bytes; ++b) code[b] = 0;
                for (int t = steps - 1; t >= stop; --t) {
                    if (pass == 1) {
                        for (int v = 0; v < V; ++v) out[row * T + (int64_t)t * V + v] = mul_rn(table[state * V + v], sc);
                        if (states) states[row * steps + t] = state;
                        if (code) {
                            // this step's symbol, most significant bit first; the first state's upper bits when a header is kept
                            for (int b = 0; b < shift; ++b) {
                                const int64_t at = header + (int64_t)t * shift + b;
                                if ((state >> (shift - 1 - b)) & 1) code[at >> 3] |= (uint8_t)(1u << (at & 7));
                            }
                            if (t == 0)
                                for (int b = 0; b < header; ++b)
                                    if ((state >> (Lbits - 1 - b)) & 1) code[b >> 3] |= (uint8_t)(1u << (b & 7));
                        }
                    }
                    if (t > stop) {
                        const long long low = state >> shift;
                        state = (long long)choices[(row * slots + (t - 1)) * G + low] * G + low;
                    }
                }
                if (pass == 0) seq_overlap[tid] = state >> shift;
            }
            __syncthreads();
        }
    }
}

// The same search for a code table with few distinct rows.  The shipped codes map 2^16 states onto about a thousand
// distinct value tuples (HYB: 2^9 lookup rows times a sign; 1MAD: a sum of four bytes), and the local cost of a state
// depends on its tuple only.  With the states' tuple numbers (`ids`, 16 bits each, the whole array in shared memory) and
// the distinct tuples, a step first forms the D local costs of every sequence (the same subtractions, products and sum
// as above, so the same bits), then every state costs one shared-memory lookup and one addition instead of a table load
// from L2 and five arithmetic instructions.  A thread takes eight neighbouring groups at a time: their tuple numbers are
// one 16-byte load and they share their predecessors' group minimum.  Results are bit for bit those of viterbi_kernel.
template <typename F, int R>
__global__ void __launch_bounds__(VT) viterbi_indexed_kernel(int64_t rows, int T, const F *__restrict__ x, const F *__restrict__ table,
                                                             const F *__restrict__ distinct, int D, const uint16_t *__restrict__ ids,
                                                             int Lbits, int shift, int V, int tail_biting, const F *__restrict__ scale,
                                                             F *__restrict__ out, int64_t *__restrict__ states, uint8_t *__restrict__ choices,
                                                             uint8_t *__restrict__ codes, int64_t code_bytes) {
    extern __shared__ __align__(16) unsigned char g2d_vsmem[];
    const int S = 1 << Lbits, G = S >> shift, H = 1 << shift;
    const int steps = T / V;
    uint16_t *id_s = reinterpret_cast<uint16_t *>(g2d_vsmem);                        // [S]
    F *B = reinterpret_cast<F *>(g2d_vsmem + (size_t)S * sizeof(uint16_t));          // [2][R][G]
    F *dist = B + (size_t)2 * R * G;                                                 // [R][D]
    __shared__ F red_val[VT / 32][R];
    __shared__ int red_arg[VT / 32][R];
    __shared__ int seq_state[R], seq_overlap[R];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t slots = steps > 1 ? steps - 1 : 1;
    for (int i = tid; i < S / 8; i += VT) reinterpret_cast<uint4 *>(id_s)[i] = reinterpret_cast<const uint4 *>(ids)[i];

    for (int64_t row0 = (int64_t)blockIdx.x * R; row0 < rows; row0 += (int64_t)gridDim.x * R) {
        if (tid < R) seq_overlap[tid] = -1;
        __syncthreads();
        for (int pass = tail_biting ? 0 : 1; pass < 2; ++pass) {
            const int half = steps / 2;
            const int roll = pass == 0 ? steps - half : 0;
            const int stop = pass == 0 ? half : 0;
            for (int t = 0; t < steps; ++t) {
                const bool last = t == steps - 1;
                const F *prev = B + (size_t)((t + 1) & 1) * R * G;
                F *next = B + (size_t)(t & 1) * R * G;
                F x0[R], x1[R];
                int ov[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int64_t row = row0 + r < rows ? row0 + r : rows - 1;
                    const F *xt = x + row * T + (int64_t)((t + roll) % steps) * V;
                    x0[r] = xt[0];
                    x1[r] = V == 2 ? xt[1] : (F)0;
                    ov[r] = seq_overlap[r];
                }
                // the local cost of every distinct tuple, for every sequence of the CTA
                for (int d = tid; d < D; d += VT) {
                    const F t0 = distinct[(int64_t)d * V], t1 = V == 2 ? distinct[(int64_t)d * V + 1] : (F)0;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const F d0 = sub_rn(t0, x0[r]);
                        F c = mul_rn(d0, d0);
                        if (V == 2) {
                            const F d1 = sub_rn(t1, x1[r]);
                            c = add_rn(c, mul_rn(d1, d1));
                        }
                        dist[r * D + d] = c;
                    }
                }
                __syncthreads();
                if (!last) {
                    // group minima of this step: eight neighbouring groups per thread and round
                    for (int g0 = tid * 8; g0 < G; g0 += VT * 8) {
                        F best[R][8];
                        int arg[R][8];
                        for (int h = 0; h < H; ++h) {
                            const uint4 packed = *reinterpret_cast<const uint4 *>(id_s + (size_t)h * G + g0);
                            const uint32_t word[4] = {packed.x, packed.y, packed.z, packed.w};
                            const int low = (h * G + g0) >> shift;  // shared by the eight groups when shift >= 3
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const int id = (word[e >> 1] >> ((e & 1) * 16)) & 0xFFFF;
                                const int low_e = shift >= 3 ? low : (h * G + g0 + e) >> shift;
#pragma unroll
                                for (int r = 0; r < R; ++r) {
                                    F c = dist[r * D + id];
                                    if (t == 0) {
                                        if (ov[r] >= 0 && low_e != ov[r]) c = pos_inf<F>();
                                    } else {
                                        c = add_rn(prev[r * G + low_e], c);
                                    }
                                    if (h == 0 || c < best[r][e]) { best[r][e] = c; arg[r][e] = h; }
                                }
                            }
                        }
#pragma unroll
                        for (int r = 0; r < R; ++r)
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                next[r * G + g0 + e] = best[r][e];
                                if (row0 + r < rows) choices[((row0 + r) * slots + t) * G + g0 + e] = (uint8_t)arg[r][e];
                            }
                    }
                    __syncthreads();
                } else {
                    // last step: first arg-min over all states, with the final mask
                    F best[R];
                    int arg[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) { best[r] = pos_inf<F>(); arg[r] = S; }
                    for (int s = tid; s < S; s += VT) {
                        const int id = id_s[s], low = s >> shift;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            F c = dist[r * D + id];
                            if (t == 0) {
                                if (ov[r] >= 0 && low != ov[r]) c = pos_inf<F>();
                            } else {
                                c = add_rn(prev[r * G + low], c);
                            }
                            if (ov[r] >= 0 && (s & (G - 1)) != ov[r]) c = pos_inf<F>();
                            if (arg[r] == S || c < best[r]) { best[r] = c; arg[r] = s; }  // ascending s: strict < keeps the first minimum
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        F b = best[r];
                        int a = arg[r];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const F ob = __shfl_xor_sync(0xffffffffu, b, o);
                            const int oa = __shfl_xor_sync(0xffffffffu, a, o);
                            if (oa < S && (a >= S || ob < b || (ob == b && oa < a))) { b = ob; a = oa; }
                        }
                        if (lane == 0) { red_val[warp][r] = b; red_arg[warp][r] = a; }
                    }
                    __syncthreads();
                    if (tid < R) {
                        F b = red_val[0][tid];
                        int a = red_arg[0][tid];
                        for (int w = 1; w < VT / 32; ++w) {
                            const F ob = red_val[w][tid];
                            const int oa = red_arg[w][tid];
                            if (oa < S && (a >= S || ob < b || (ob == b && oa < a))) { b = ob; a = oa; }
                        }
                        seq_state[tid] = a;
                    }
                    __syncthreads();
                }
            }
            // ---- walk back: thread r follows sequence r ----
            if (tid < R && row0 + tid < rows) {
                const int64_t row = row0 + tid;
                long long state = seq_state[tid];
                const F sc = scale ? scale[row] : (F)1;
                uint8_t *code = (pass == 1 && codes) ? codes + row * code_bytes : nullptr;
                const int header = tail_biting ? 0 : Lbits - shift;
                if (code)
                    for (int64_t b = 0; b < code_bytes; ++b) code[b] = 0;
                for (int t = steps - 1; t >= stop; --t) {
                    if (pass == 1) {
                        for (int v = 0; v < V; ++v) out[row * T + (int64_t)t * V + v] = mul_rn(table[state * V + v], sc);
                        if (states) states[row * steps + t] = state;
                        if (code) {
                            for (int b = 0; b < shift; ++b) {
                                const int64_t at = header + (int64_t)t * shift + b;
                                if ((state >> (shift - 1 - b)) & 1) code[at >> 3] |= (uint8_t)(1u << (at & 7));
                            }
                            if (t == 0)
                                for (int b = 0; b < header; ++b)
                                    if ((state >> (Lbits - 1 - b)) & 1) code[b >> 3] |= (uint8_t)(1u << (b & 7));
                        }
                    }
                    if (t > stop) {
                        const long long low = state >> shift;
                        state = (long long)choices[(row * slots + (t - 1)) * G + low] * G + low;
                    }
                }
                if (pass == 0) seq_overlap[tid] = (int)(state >> shift);
            }
            __syncthreads();
        }
    }
}

// Values (and optionally states) of stored bit strings: one thread per (sequence, step) rebuilds the state from the L
// bits of the string that end with the step's symbol.
template <typename F>
__global__ void trellis_decode_kernel(int64_t rows, int T, const uint8_t *__restrict__ codes, int64_t code_bytes, const F *__restrict__ table,
                                      int Lbits, int shift, int V, int tail_biting, const F *__restrict__ scale, F *__restrict__ out,
                                      int64_t *__restrict__ states) {
    const int steps = T / V;
    const int header = tail_biting ? 0 : Lbits - shift;
    const int64_t bits = header + (int64_t)steps * shift, total = rows * steps;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / steps;
        const int t = (int)(idx % steps);
        const uint8_t *code = codes + row * code_bytes;
        const int64_t end = header + (int64_t)(t + 1) * shift;  // one past the last bit of the state
        long long state = 0;
        for (int b = 0; b < Lbits; ++b) {
            int64_t at = end - Lbits + b;
            if (at < 0) at += bits;  // tail-biting only: a string with a header always reaches back far enough
            state = (state << 1) | ((code[at >> 3] >> (at & 7)) & 1);
        }
        const F sc = scale ? scale[row] : (F)1;
        for (int v = 0; v < V; ++v) out[row * T + (int64_t)t * V + v] = mul_rn(table[state * V + v], sc);
        if (states) states[row * steps + t] = state;
    }
}

template <typename F, int R>
static int launch_viterbi(int64_t rows, int T, const void *x, const void *table, int L, int K, int V, int tail, const void *scale,
                          void *out, int64_t *states, void *workspace, uint8_t *codes, int64_t code_bytes, cudaStream_t st) {
    static PerDeviceOnce configured;
    const int64_t G = ((int64_t)1 << L) >> (K * V);
    const size_t smem = sizeof(F) * 2 * R * (size_t)G;
    if (configured.run([&] { return cudaFuncSetAttribute(viterbi_kernel<F, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess; }) != G2D_OK)
        return G2D_ERR_CUDA;
    int64_t blocks = ceil_div(rows, R);
    if (blocks > 148 * 8) blocks = 148 * 8;
    viterbi_kernel<F, R><<<(unsigned)blocks, VT, smem, st>>>(rows, T, (const F *)x, (const F *)table, L, K * V, V, tail, (const F *)scale,
                                                             (F *)out, states, (uint8_t *)workspace, codes, code_bytes);
    return check_launch();
}

template <typename F>
static int trellis_dispatch(int64_t rows, int T, const void *x, const void *table, int L, int K, int V, int tail, const void *scale,
                            void *out, int64_t *states, void *workspace, uint8_t *codes, int64_t code_bytes, cudaStream_t st) {
    const int64_t G = ((int64_t)1 << L) >> (K * V);
    const size_t per_seq = sizeof(F) * 2 * (size_t)G;
    const size_t budget = 200 * 1024;
    if (per_seq > budget) return G2D_ERR_TOO_LARGE;
    // More sequences per CTA share each table read and its address arithmetic, fewer finish a short coarse anti-diagonal
    // sooner.  Measured on B200 (HYB, L = 16, T = 256) one wave of CTAs with 1 / 2 / 4 sequences each takes 1.6 / 2.4 /
    // 4.3 ms, so the fewest sequences per CTA that still fit one wave of SMs win, and four per CTA beyond that.
    int R = 1;
    if (rows > 148 && 2 * per_seq <= budget) R = 2;
    if (rows > 2 * 148 && 4 * per_seq <= budget) R = 4;
    switch (R) {
    case 4: return launch_viterbi<F, 4>(rows, T, x, table, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
    case 2: return launch_viterbi<F, 2>(rows, T, x, table, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
    default: return launch_viterbi<F, 1>(rows, T, x, table, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
    }
}

int64_t trellis_code_bytes(int T, int L, int K, int V, int tail_biting) {
    const int64_t bits = (tail_biting ? 0 : L - K * V) + (int64_t)(T / V) * K * V;
    return (bits + 7) / 8;
}

size_t trellis_scratch_bytes(int dtype, int64_t rows, int T, int L, int K, int V) {
    const int64_t steps = T / V, slots = steps > 1 ? steps - 1 : 1, G = ((int64_t)1 << L) >> (K * V);
    (void)dtype;
    return ((size_t)rows * slots * G + 255) & ~(size_t)255;
}

template <typename F, int R>
static int launch_viterbi_indexed(int64_t rows, int T, const void *x, const void *table, const TrellisIndex &index, int L, int K, int V, int tail,
                                  const void *scale, void *out, int64_t *states, void *workspace, uint8_t *codes, int64_t code_bytes, cudaStream_t st) {
    static PerDeviceOnce configured;
    const int64_t S = (int64_t)1 << L, G = S >> (K * V);
    const size_t smem = (size_t)S * sizeof(uint16_t) + sizeof(F) * (2 * R * (size_t)G + (size_t)R * index.count);
    if (configured.run([&] { return cudaFuncSetAttribute(viterbi_indexed_kernel<F, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) == cudaSuccess; }) != G2D_OK)
        return G2D_ERR_CUDA;
    int64_t blocks = ceil_div(rows, R);
    if (blocks > 148 * 8) blocks = 148 * 8;
    viterbi_indexed_kernel<F, R><<<(unsigned)blocks, VT, smem, st>>>(rows, T, (const F *)x, (const F *)table, (const F *)index.distinct, index.count,
                                                                     index.ids, L, K * V, V, tail, (const F *)scale, (F *)out, states,
                                                                     (uint8_t *)workspace, codes, code_bytes);
    return check_launch();
}

// The indexed search serves tables of up to 2^16 states whose distinct rows fit shared memory beside the group minima, and
// only calls of at most one sequence per SM.  Measured on B200 (HYB, L = 16, T = 256): 148 sequences take 1.58 ms against
// 1.87 ms for the search that reads the table from L2, but with two sequences per CTA the random look-ups of the local
// costs collide in the shared-memory banks (256 sequences: 3.6 ms against 2.6 ms; 4096: 49 ms against 30 ms), so larger
// calls keep the other kernel.
template <typename F>
static int indexed_sequences_per_cta(const TrellisIndex *index, int64_t rows, int L, int K, int V) {
    if (index == nullptr || index->ids == nullptr || index->distinct == nullptr || index->count <= 0) return 0;
    const int64_t S = (int64_t)1 << L, G = S >> (K * V);
    if (L > 16 || G < 8 || S < 8 || rows > 148) return 0;
    const size_t bytes = (size_t)S * 2 + sizeof(F) * (2 * (size_t)G + (size_t)index->count);
    return bytes <= 216 * 1024 ? 1 : 0;
}

int launch_trellis(int dtype, int64_t rows, int T, const void *x, const void *table, int L, int K, int V, int tail, const void *scale,
                   void *out, int64_t *states, void *workspace, uint8_t *codes, cudaStream_t st, const TrellisIndex *index) {
    const int64_t code_bytes = trellis_code_bytes(T, L, K, V, tail);
    const int R = dtype == G2D_F32 ? indexed_sequences_per_cta<float>(index, rows, L, K, V) : indexed_sequences_per_cta<double>(index, rows, L, K, V);
    if (R == 1 && dtype == G2D_F32) return launch_viterbi_indexed<float, 1>(rows, T, x, table, *index, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
    if (R == 1) return launch_viterbi_indexed<double, 1>(rows, T, x, table, *index, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
    return dtype == G2D_F32 ? trellis_dispatch<float>(rows, T, x, table, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st)
                            : trellis_dispatch<double>(rows, T, x, table, L, K, V, tail, scale, out, states, workspace, codes, code_bytes, st);
}

}  // namespace g2d

using namespace g2d;

static int trellis_check(int dtype, int64_t rows, int32_t T, int32_t L, int32_t K, int32_t V) {
    if (dtype != G2D_F32 && dtype != G2D_F64) return G2D_ERR_BAD_ARGUMENT;
    if (rows < 0 || T <= 0 || V < 1 || V > 2 || K < 1 || K * V > 8 || L < K * V || L > 24 || T % V != 0) return G2D_ERR_BAD_ARGUMENT;
    return G2D_OK;
}

extern "C" int g2d_trellis_workspace_bytes(int dtype, int64_t rows, int32_t T, int32_t L, int32_t K, int32_t V, size_t *bytes) {
    const int status = trellis_check(dtype, rows, T, L, K, V);
    if (status != G2D_OK || !bytes) return status != G2D_OK ? status : G2D_ERR_BAD_ARGUMENT;
    *bytes = trellis_scratch_bytes(dtype, rows, T, L, K, V);
    return G2D_OK;
}

extern "C" int g2d_trellis_quantize(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                                    int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states,
                                    void *workspace, size_t workspace_bytes, void *stream) {
    const int status = trellis_check(dtype, rows, T, L, K, V);
    if (status != G2D_OK) return status;
    if (rows == 0) return G2D_OK;
    if (!x || !table || !out) return G2D_ERR_BAD_ARGUMENT;
    size_t need = 0;
    g2d_trellis_workspace_bytes(dtype, rows, T, L, K, V, &need);
    if (!workspace || workspace_bytes < need) return G2D_ERR_WORKSPACE;
    return launch_trellis(dtype, rows, T, x, table, L, K, V, tail_biting, scale, out, states, workspace, nullptr, (cudaStream_t)stream);
}

extern "C" int g2d_trellis_code_bytes(int32_t T, int32_t L, int32_t K, int32_t V, int32_t tail_biting, int64_t *bytes) {
    const int status = trellis_check(G2D_F32, 0, T, L, K, V);
    if (status != G2D_OK || !bytes) return status != G2D_OK ? status : G2D_ERR_BAD_ARGUMENT;
    *bytes = trellis_code_bytes(T, L, K, V, tail_biting);
    return G2D_OK;
}

extern "C" int g2d_trellis_quantize_packed(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                                           int32_t V, int32_t tail_biting, const void *scale, void *out, uint8_t *codes,
                                           void *workspace, size_t workspace_bytes, void *stream) {
    const int status = trellis_check(dtype, rows, T, L, K, V);
    if (status != G2D_OK) return status;
    if (rows == 0) return G2D_OK;
    if (!x || !table || !out || !codes) return G2D_ERR_BAD_ARGUMENT;
    if (!tail_biting && (int64_t)(T / V) * K * V + L - K * V < L) return G2D_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < trellis_scratch_bytes(dtype, rows, T, L, K, V)) return G2D_ERR_WORKSPACE;
    return launch_trellis(dtype, rows, T, x, table, L, K, V, tail_biting, scale, out, nullptr, workspace, codes, (cudaStream_t)stream);
}

extern "C" int g2d_trellis_quantize_indexed(int dtype, int64_t rows, int32_t T, const void *x, const void *table, int32_t L, int32_t K,
                                            int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states, uint8_t *codes,
                                            const void *distinct, int32_t distinct_count, const uint16_t *ids, void *workspace,
                                            size_t workspace_bytes, void *stream) {
    const int status = trellis_check(dtype, rows, T, L, K, V);
    if (status != G2D_OK) return status;
    if (rows == 0) return G2D_OK;
    if (!x || !table || !out || !distinct || !ids || distinct_count <= 0 || distinct_count > 65536) return G2D_ERR_BAD_ARGUMENT;
    if (((uintptr_t)ids & 15) != 0) return G2D_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < trellis_scratch_bytes(dtype, rows, T, L, K, V)) return G2D_ERR_WORKSPACE;
    const TrellisIndex index{distinct, ids, distinct_count};
    return launch_trellis(dtype, rows, T, x, table, L, K, V, tail_biting, scale, out, states, workspace, codes, (cudaStream_t)stream, &index);
}

extern "C" int g2d_trellis_decode(int dtype, int64_t rows, int32_t T, const uint8_t *codes, const void *table, int32_t L, int32_t K,
                                  int32_t V, int32_t tail_biting, const void *scale, void *out, int64_t *states, void *stream) {
    const int status = trellis_check(dtype, rows, T, L, K, V);
    if (status != G2D_OK) return status;
    if (rows == 0) return G2D_OK;
    if (!codes || !table || !out) return G2D_ERR_BAD_ARGUMENT;
    if (tail_biting && (int64_t)(T / V) * K * V < L) return G2D_ERR_UNSUPPORTED;  // a string shorter than one state does not determine it
    const int64_t bytes = trellis_code_bytes(T, L, K, V, tail_biting), total = rows * (T / V);
    int64_t blocks = ceil_div(total, 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == G2D_F32)
        trellis_decode_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(rows, T, codes, bytes, (const float *)table, L, K * V, V, tail_biting,
                                                                      (const float *)scale, (float *)out, states);
    else
        trellis_decode_kernel<double><<<(unsigned)blocks, 256, 0, st>>>(rows, T, codes, bytes, (const double *)table, L, K * V, V, tail_biting,
                                                                       (const double *)scale, (double *)out, states);
    return check_launch();
}
