// Row-wise kernels beside the RMSNorm of elementwise.cu: a layer norm with weight and bias on the
// residual stream, an RMS norm of plain rows (whole rows or groups of a row, any element type), the
// PolyNorm activation, the gate of a per-layer token input, its normalised addition to the stream, a
// weighted sum of kept copies of the stream, and an add-and-cast of the stream.
//
// Everything that is summed over a row (means, variances, mean squares) is 32-bit; the residual stream
// is 32-bit in every engine dtype. Each reduction's order depends on the row's width only, so a row's
// result does not depend on what else the launch holds.
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

// ---------------------------------------------------------------- residual add + layer norm
// One block per output row r; source row s = row_index ? row_index[r] : r.
//   d = delta[s], or with delta_weight the delta's own layer norm without bias:
//       d = (delta[s] - mean(delta[s])) / sqrt(mean((delta[s] - mean)^2) + delta_eps) * delta_weight
//   v = residual[s] + d (delta optional); if write_residual: residual[s] = v
//   y[r] = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w + b        (y optional: only the sum is formed)
// The row is staged in shared memory; the variance is taken of the deviations (second pass).
template <typename TD, typename TY>
__global__ void __launch_bounds__(ROW_THREADS)
add_layernorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const float* __restrict__ weight,
                     const float* __restrict__ bias, TY* __restrict__ y, const int* __restrict__ row_index,
                     int hidden, float eps, int write_residual, const float* __restrict__ delta_weight,
                     float delta_eps) {
    extern __shared__ float staged[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float* h = residual + s * hidden;
    float delta_mean = 0.f, delta_inv = 1.f;
    if (delta && delta_weight) {
        float* d = staged + hidden;
        float sum = 0.f;
        for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
            const float value = to_float(delta[s * hidden + c]);
            d[c] = value;
            sum += value;
        }
        delta_mean = block_sum<ROW_THREADS>(sum, scratch) / (float)hidden;
        float square = 0.f;
        for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
            const float deviation = d[c] - delta_mean;
            square = fmaf(deviation, deviation, square);
        }
        delta_inv = 1.0f / sqrtf(block_sum<ROW_THREADS>(square, scratch) / (float)hidden + delta_eps);
    }
    float sum = 0.f;
    for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
        float value = h[c];
        if (delta) {
            if (delta_weight) value += (staged[hidden + c] - delta_mean) * delta_inv * delta_weight[c];
            else value += to_float(delta[s * hidden + c]);
        }
        if (write_residual) h[c] = value;
        staged[c] = value;
        sum += value;
    }
    if (!y) return;
    const float mean = block_sum<ROW_THREADS>(sum, scratch) / (float)hidden;
    float square = 0.f;
    for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
        const float deviation = staged[c] - mean;
        square = fmaf(deviation, deviation, square);
    }
    const float variance = block_sum<ROW_THREADS>(square, scratch) / (float)hidden;
    const float inv = 1.0f / sqrtf(variance + eps);
    TY* out = y + (long long)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += ROW_THREADS)
        out[c] = from_float<TY>((staged[c] - mean) * inv * weight[c] + (bias ? bias[c] : 0.f));
}

// ---------------------------------------------------------------- a gate per head; an activation; a vector on every row
// x[r, h, :] *= sigmoid(gate[r, h]) for x [rows, heads, width] and gate logits [rows, heads] (row stride ldg);
// the sigmoid and the product are 32-bit.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, long long ldx, const T* __restrict__ gate, long long ldg,
                                 long long total, int heads, int width) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at >= total) return;
    const int per_row = heads * width;
    const long long row = at / per_row;
    const int c = (int)(at - row * per_row);
    const float g = to_float(gate[row * ldg + c / width]);
    T* value = x + row * ldx + c;
    *value = from_float<T>(to_float(*value) / (1.0f + expf(-g)));
}

// out = 0.5 z (1 + erf(z / sqrt 2)), element by element.
template <typename T>
__global__ void gelu_kernel(const T* __restrict__ z, T* __restrict__ out, long long total) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at >= total) return;
    const float v = to_float(z[at]);
    out[at] = from_float<T>(0.5f * v * (1.0f + erff(v * 0.70710678118654752440f)));
}

// The same for bfloat16, eight elements (16 bytes) a thread; `groups` = total / 8.
__global__ void gelu_bf16x8_kernel(const bf16* __restrict__ z, bf16* __restrict__ out, long long groups) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at >= groups) return;
    uint4 raw = *reinterpret_cast<const uint4*>(z + at * 8);
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 v = __bfloat1622float2(pairs[k]);
        pairs[k] = __floats2bfloat162_rn(0.5f * v.x * (1.0f + erff(v.x * 0.70710678118654752440f)),
                                         0.5f * v.y * (1.0f + erff(v.y * 0.70710678118654752440f)));
    }
    *reinterpret_cast<uint4*>(out + at * 8) = raw;
}

// x *= factor, element by element (x 32-bit, in place).
__global__ void scale_kernel(float* __restrict__ x, long long total, float factor) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at < total) x[at] *= factor;
}

// x[r, :] += vector (x 32-bit, in place).
template <typename TW>
__global__ void add_vector_kernel(float* __restrict__ x, const TW* __restrict__ vector, long long total, int hidden) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at >= total) return;
    x[at] += to_float(vector[at % hidden]);
}

// ---------------------------------------------------------------- RMS norm of groups of plain rows
// One warp per (row, group): out[row, g*width + c] = x[row, g*width + c] / sqrt(mean_c(x^2) + eps) * w[c]
// (w optional, shared by the groups).
template <typename T>
__global__ void __launch_bounds__(128)
rms_rows_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ out, long long ldo,
                const float* __restrict__ weight, int rows, int groups, int width, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)rows * groups) return;
    const int row = (int)(item / groups), group = (int)(item - (long long)row * groups);
    const T* source = x + row * ldx + (long long)group * width;
    T* target = out + row * ldo + (long long)group * width;
    float square = 0.f;
    for (int c = lane; c < width; c += 32) {
        const float value = to_float(source[c]);
        square = fmaf(value, value, square);
    }
    const float inv = 1.0f / sqrtf(warp_sum(square) / (float)width + eps);
    for (int c = lane; c < width; c += 32)
        target[c] = from_float<T>(to_float(source[c]) * inv * (weight ? weight[c] : 1.f));
}

// ---------------------------------------------------------------- PolyNorm
// out = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e over a row of `width` values, powers
// element by element, rms(u) = sqrt(mean(u^2) + eps).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
poly_norm_kernel(const T* __restrict__ z, T* __restrict__ out, const float* __restrict__ coefficients, int width,
                 float eps) {
    __shared__ float scratch[32];
    const long long row = blockIdx.x;
    const T* source = z + row * width;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
        const float v = to_float(source[c]);
        const float v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    const float r1 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s2, scratch) / (float)width + eps);
    const float r2 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s4, scratch) / (float)width + eps);
    const float r3 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s6, scratch) / (float)width + eps);
    const float a = coefficients[0] * r1, b = coefficients[1] * r2, c3 = coefficients[2] * r3, e = coefficients[3];
    T* target = out + row * width;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
        const float v = to_float(source[c]);
        const float v2 = v * v;
        target[c] = from_float<T>(a * v + b * v2 + c3 * v2 * v + e);
    }
}

// The same for bfloat16 rows whose width is a multiple of 8: 16 bytes a load (the second pass finds the row in
// the caches). The sums are added in another order than above, fixed by the width.
__global__ void __launch_bounds__(ROW_THREADS)
poly_norm_bf16x8_kernel(const bf16* __restrict__ z, bf16* __restrict__ out, const float* __restrict__ coefficients,
                        int width, float eps) {
    __shared__ float scratch[32];
    const long long row = blockIdx.x;
    const uint4* source = reinterpret_cast<const uint4*>(z + row * width);
    const int pieces = width >> 3;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll 4
    for (int i = threadIdx.x; i < pieces; i += ROW_THREADS) {
        const uint4 piece = source[i];
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&piece);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 v = __bfloat1622float2(pairs[e]);
            const float x2 = v.x * v.x, y2 = v.y * v.y, x3 = x2 * v.x, y3 = y2 * v.y;
            s2 += x2 + y2;
            s4 = fmaf(x2, x2, fmaf(y2, y2, s4));
            s6 = fmaf(x3, x3, fmaf(y3, y3, s6));
        }
    }
    const float r1 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s2, scratch) / (float)width + eps);
    const float r2 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s4, scratch) / (float)width + eps);
    const float r3 = 1.0f / sqrtf(block_sum<ROW_THREADS>(s6, scratch) / (float)width + eps);
    const float a = coefficients[0] * r1, b = coefficients[1] * r2, c3 = coefficients[2] * r3, e0 = coefficients[3];
    uint4* target = reinterpret_cast<uint4*>(out + row * width);
#pragma unroll 4
    for (int i = threadIdx.x; i < pieces; i += ROW_THREADS) {
        uint4 piece = source[i];
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&piece);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 v = __bfloat1622float2(pairs[e]);
            pairs[e] = __floats2bfloat162_rn(fmaf(fmaf(fmaf(c3, v.x, b), v.x, a), v.x, e0),
                                             fmaf(fmaf(fmaf(c3, v.y, b), v.y, a), v.y, e0));
        }
        target[i] = piece;
    }
}

// ---------------------------------------------------------------- gate of a per-layer token input
__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// g[r, c] = gelu_tanh(gate[r, c]) * table[token[r], offset + c], c < dim.
template <typename T, typename TW>
__global__ void token_gate_kernel(const T* __restrict__ gate, T* __restrict__ out, const TW* __restrict__ table,
                                  long long table_ld, int offset, const int* __restrict__ tokens, int vocab,
                                  long long total, int dim) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / dim;
    const int c = (int)(index - row * dim);
    const int token = tokens[row];
    const float e = token >= 0 && token < vocab ? to_float(table[token * table_ld + offset + c]) : 0.f;
    out[index] = from_float<T>(gelu_tanh(to_float(gate[index])) * e);
}

// ---------------------------------------------------------------- normalised addition, weighted sum of kept streams
// One block per row r:
//   x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w                       (y may be null: nothing is added)
//   if mixed: mixed[r] = sum_{j < count} mix[j] * kept[j][r]           kept[j] = kept + j * kept_stride
// (x itself is usually the last of the kept streams: it is written before it is summed.)
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
add_normed_mix_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ weight, int hidden,
                      float eps, const float* __restrict__ kept, long long kept_stride, const float* __restrict__ mix,
                      int count, float* __restrict__ mixed) {
    __shared__ float scratch[32];
    const long long r = blockIdx.x;
    float* row = x + r * hidden;
    if (y) {
        const T* addend = y + r * hidden;
        float square = 0.f;
        for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
            const float v = to_float(addend[c]);
            square = fmaf(v, v, square);
        }
        const float inv = 1.0f / sqrtf(block_sum<ROW_THREADS>(square, scratch) / (float)hidden + eps);
        for (int c = threadIdx.x; c < hidden; c += ROW_THREADS)   // a thread reads below what it wrote itself
            row[c] += to_float(addend[c]) * inv * weight[c];
    }
    if (!mixed) return;
    for (int c = threadIdx.x; c < hidden; c += ROW_THREADS) {
        float total = 0.f;
        for (int j = 0; j < count; ++j) total = fmaf(mix[j], kept[j * kept_stride + r * hidden + c], total);
        mixed[r * hidden + c] = total;
    }
}

// x += delta (32-bit, in place; delta optional) and, if asked, a copy of x in T.
template <typename TD, typename T>
__global__ void add_cast_kernel(float* __restrict__ x, const TD* __restrict__ delta, T* __restrict__ copy,
                                long long total) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    float value = x[index];
    if (delta) {
        value += to_float(delta[index]);
        x[index] = value;
    }
    if (copy) copy[index] = from_float<T>(value);
}

}  // namespace

KIDI_API int kidi_add_layernorm(float* residual, const void* delta, int delta_dtype, const float* weight,
                                const float* bias, void* y, int y_dtype, const int* row_index, int rows, int hidden,
                                float eps, int write_residual, const float* delta_weight, float delta_eps,
                                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (delta_dtype == KIDI_NONE) { delta = nullptr; delta_dtype = KIDI_F32; }
    if (y_dtype == KIDI_NONE) { y = nullptr; y_dtype = KIDI_F32; }
    if (!delta) delta_weight = nullptr;
    const size_t shared = (size_t)hidden * sizeof(float) * (delta_weight ? 2 : 1);
    if (hidden <= 0 || shared > 200 * 1024) return KIDI_REFUSED_SIZE;
#define KIDI_CASE(D, TD, Y, TY)                                                                                    \
    if (delta_dtype == D && y_dtype == Y) {                                                                        \
        auto kernel = add_layernorm_kernel<TD, TY>;                                                                \
        if (shared > 48 * 1024) {                                                                                  \
            cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared); \
            if (status != cudaSuccess) return (int)status;                                                         \
        }                                                                                                          \
        return kidi_launch(kernel, rows, ROW_THREADS, shared, stream, residual, (const TD*)delta, weight, bias,    \
                           (TY*)y, row_index, hidden, eps, write_residual, delta_weight, delta_eps);               \
    }
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_head_gate(void* x, long long ldx, const void* gate, long long ldg, int dtype, int rows, int heads,
                            int width, cudaStream_t stream) {
    const long long total = (long long)rows * heads * width;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(head_gate_kernel<float>, blocks, 256, 0, stream, (float*)x, ldx,
                                              (const float*)gate, ldg, total, heads, width);
    if (dtype == KIDI_BF16) return kidi_launch(head_gate_kernel<bf16>, blocks, 256, 0, stream, (bf16*)x, ldx,
                                               (const bf16*)gate, ldg, total, heads, width);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_gelu(const void* z, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(gelu_kernel<float>, blocks, 256, 0, stream, (const float*)z, (float*)out, total);
    if (dtype == KIDI_BF16 && !(total & 7) && !((uintptr_t)z & 15) && !((uintptr_t)out & 15))
        return kidi_launch(gelu_bf16x8_kernel, (unsigned)(((total >> 3) + 255) / 256), 256, 0, stream, (const bf16*)z,
                           (bf16*)out, total >> 3);
    if (dtype == KIDI_BF16) return kidi_launch(gelu_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)z, (bf16*)out, total);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_scale(float* x, long long total, float factor, cudaStream_t stream) {
    if (total <= 0) return 0;
    return kidi_launch(scale_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, total, factor);
}

KIDI_API int kidi_add_vector(float* x, const void* vector, int vector_dtype, int rows, int hidden, cudaStream_t stream) {
    const long long total = (long long)rows * hidden;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (vector_dtype == KIDI_F32) return kidi_launch(add_vector_kernel<float>, blocks, 256, 0, stream, x, (const float*)vector, total, hidden);
    if (vector_dtype == KIDI_BF16) return kidi_launch(add_vector_kernel<bf16>, blocks, 256, 0, stream, x, (const bf16*)vector, total, hidden);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_rms_rows(const void* x, long long ldx, void* out, long long ldo, int dtype, const float* weight,
                           int rows, int groups, int width, float eps, cudaStream_t stream) {
    if (rows <= 0 || groups <= 0) return 0;
    if (width <= 0) return KIDI_REFUSED_SIZE;
    const long long items = (long long)rows * groups;
    if ((items + 3) / 4 > 0x7fffffffLL) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == KIDI_F32)
        return kidi_launch(rms_rows_kernel<float>, blocks, 128, 0, stream, (const float*)x, ldx, (float*)out, ldo,
                           weight, rows, groups, width, eps);
    if (dtype == KIDI_BF16)
        return kidi_launch(rms_rows_kernel<bf16>, blocks, 128, 0, stream, (const bf16*)x, ldx, (bf16*)out, ldo, weight,
                           rows, groups, width, eps);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_poly_norm(const void* z, void* out, int dtype, const float* coefficients, int rows, int width,
                            float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32)
        return kidi_launch(poly_norm_kernel<float>, rows, ROW_THREADS, 0, stream, (const float*)z, (float*)out,
                           coefficients, width, eps);
    if (dtype == KIDI_BF16) {
        if (!(width & 7) && !((uintptr_t)z & 15) && !((uintptr_t)out & 15))
            return kidi_launch(poly_norm_bf16x8_kernel, rows, ROW_THREADS, 0, stream, (const bf16*)z, (bf16*)out,
                               coefficients, width, eps);
        return kidi_launch(poly_norm_kernel<bf16>, rows, ROW_THREADS, 0, stream, (const bf16*)z, (bf16*)out,
                           coefficients, width, eps);
    }
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_token_gate(const void* gate, void* out, int dtype, const void* table, int table_dtype,
                             long long table_ld, int offset, const int* tokens, int vocab, int rows, int dim,
                             cudaStream_t stream) {
    const long long total = (long long)rows * dim;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
#define KIDI_CASE(D, T, W, TW)                                                                                 \
    if (dtype == D && table_dtype == W)                                                                        \
        return kidi_launch(token_gate_kernel<T, TW>, blocks, 256, 0, stream, (const T*)gate, (T*)out,          \
                           (const TW*)table, table_ld, offset, tokens, vocab, total, dim);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_add_normed_mix(float* x, const void* y, int y_dtype, const float* weight, int rows, int hidden,
                                 float eps, const float* kept, long long kept_stride, const float* mix, int count,
                                 float* mixed, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (mixed && (count <= 0 || !kept || !mix)) || (y && !weight)) return KIDI_REFUSED_SIZE;
    if (y_dtype == KIDI_NONE) { y = nullptr; y_dtype = KIDI_F32; }
    if (y_dtype == KIDI_F32)
        return kidi_launch(add_normed_mix_kernel<float>, rows, ROW_THREADS, 0, stream, x, (const float*)y, weight,
                           hidden, eps, kept, kept_stride, mix, count, mixed);
    if (y_dtype == KIDI_BF16)
        return kidi_launch(add_normed_mix_kernel<bf16>, rows, ROW_THREADS, 0, stream, x, (const bf16*)y, weight, hidden,
                           eps, kept, kept_stride, mix, count, mixed);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_add_cast(float* x, const void* delta, int delta_dtype, void* copy, int copy_dtype, long long total,
                           cudaStream_t stream) {
    if (total <= 0) return 0;
    if (delta_dtype == KIDI_NONE) { delta = nullptr; delta_dtype = KIDI_F32; }
    if (copy_dtype == KIDI_NONE) { copy = nullptr; copy_dtype = KIDI_F32; }
    const unsigned blocks = (unsigned)((total + 255) / 256);
#define KIDI_CASE(D, TD, C, T)                                                                                  \
    if (delta_dtype == D && copy_dtype == C)                                                                    \
        return kidi_launch(add_cast_kernel<TD, T>, blocks, 256, 0, stream, x, (const TD*)delta, (T*)copy, total);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------- rows of a table added to the stream
// x[r, :] += table[index[r], :] * scale (x 32-bit, in place): a learned vector per position, say.
// Rows whose index lies outside the table are left as they are.
template <typename TW>
__global__ void add_table_rows_kernel(float* __restrict__ x, const TW* __restrict__ table, const int* __restrict__ index,
                                      long long total, int hidden, int table_rows, float scale) {
    const long long at = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (at >= total) return;
    const long long row = at / hidden;
    const int c = (int)(at - row * hidden);
    const int source = index[row];
    if (source < 0 || source >= table_rows) return;
    x[at] += to_float(table[(long long)source * hidden + c]) * scale;
}

KIDI_API int kidi_add_table_rows(float* x, const void* table, int table_dtype, const int* index, int rows, int hidden,
                                 int table_rows, float scale, cudaStream_t stream) {
    const long long total = (long long)rows * hidden;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (table_dtype == KIDI_F32)
        return kidi_launch(add_table_rows_kernel<float>, blocks, 256, 0, stream, x, (const float*)table, index, total,
                           hidden, table_rows, scale);
    if (table_dtype == KIDI_BF16)
        return kidi_launch(add_table_rows_kernel<bf16>, blocks, 256, 0, stream, x, (const bf16*)table, index, total,
                           hidden, table_rows, scale);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------- a bounded gate
// gate_up [rows, 2 * inter] (gate columns, then up columns):
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + up_shift)
template <typename T>
__global__ void bounded_gate_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter,
                                    float limit, float alpha, float up_shift) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / inter;
    const int c = (int)(index - row * inter);
    const float gate = fminf(to_float(gate_up[row * 2 * inter + c]), limit);
    const float up = fminf(fmaxf(to_float(gate_up[row * 2 * inter + inter + c]), -limit), limit);
    out[index] = from_float<T>(gate / (1.0f + expf(-alpha * gate)) * (up + up_shift));
}

// The same for bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) a thread.
__global__ void bounded_gate_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, long long groups,
                                           int inter, float limit, float alpha, float up_shift) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= groups) return;
    const int per_row = inter >> 3;
    const long long row = index / per_row;
    const int c = (int)(index - row * per_row) << 3;
    const uint4 gate = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + c);
    const uint4 up = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + c);
    const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&gate);
    const __nv_bfloat162* u = reinterpret_cast<const __nv_bfloat162*>(&up);
    uint4 result;
    __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 gv = __bfloat1622float2(g[i]), uv = __bfloat1622float2(u[i]);
        gv.x = fminf(gv.x, limit); gv.y = fminf(gv.y, limit);
        uv.x = fminf(fmaxf(uv.x, -limit), limit); uv.y = fminf(fmaxf(uv.y, -limit), limit);
        r[i] = __floats2bfloat162_rn(gv.x / (1.0f + expf(-alpha * gv.x)) * (uv.x + up_shift),
                                     gv.y / (1.0f + expf(-alpha * gv.y)) * (uv.y + up_shift));
    }
    *reinterpret_cast<uint4*>(out + row * inter + c) = result;
}

KIDI_API int kidi_bounded_gate(const void* gate_up, void* out, int dtype, int rows, int inter, float limit, float alpha,
                               float up_shift, cudaStream_t stream) {
    const long long total = (long long)rows * inter;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32)
        return kidi_launch(bounded_gate_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, total,
                           inter, limit, alpha, up_shift);
    if (dtype == KIDI_BF16) {
        if (!(inter & 7) && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
            const long long groups = total >> 3;
            return kidi_launch(bounded_gate_bf16x8_kernel, (unsigned)((groups + 255) / 256), 256, 0, stream,
                               (const bf16*)gate_up, (bf16*)out, groups, inter, limit, alpha, up_shift);
        }
        return kidi_launch(bounded_gate_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, total,
                           inter, limit, alpha, up_shift);
    }
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------- bounded logits
// x <- cap * tanh(x / cap), 32-bit, in place.
__global__ void tanh_cap_kernel(float* __restrict__ x, long long total, float cap) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index < total) x[index] = cap * tanhf(x[index] / cap);
}

KIDI_API int kidi_tanh_cap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    return kidi_launch(tanh_cap_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, total, cap);
}
