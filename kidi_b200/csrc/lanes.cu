// A residual stream kept as several lanes (copies that layers read as one weighted sum and write back
// through a small mixing matrix), and a few row-wise kernels of mixers that run side by side.
//
//   lanes_rmsnorm:    u = sum_s read[s] * lane_s (read absent: the plain sum);  y = u / sqrt(mean(u^2) + eps) * w
//   lanes_mix:        lane'_t = sum_s mix[s, t] * lane_s + write[t] * y          (all lanes at once, from the old ones)
//   normed_pair_sum:  z = ca * a / rms(a) * wa + cb * b / rms(b) * wb
//   sigmoid_gate:     x <- x * sigmoid(g), element by element
//   relu_squared:     z -> max(z, 0)^2
//
// The lanes, every weighted sum of them and every mean square are 32-bit. A sum over lanes runs in the
// order of the lanes and a row's reduction in an order that depends on its width only, so a row's result
// does not depend on what else the launch holds.
#include "common.cuh"

namespace {

constexpr int LANE_THREADS = 256;
constexpr int MAX_LANES = 8;

// One block per output row r; source row s = row_index ? row_index[r] : r. `lanes` + l * lane_stride is lane l
// (a stride of 0: every lane is the same matrix). weight null: y = u, not normalised.
template <typename TW, typename TY>
__global__ void __launch_bounds__(LANE_THREADS)
lanes_rmsnorm_kernel(const float* __restrict__ lanes, long long lane_stride, int count, const float* __restrict__ read,
                     const TW* __restrict__ weight, TY* __restrict__ y, const int* __restrict__ row_index, int hidden,
                     float eps) {
    extern __shared__ float staged[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float square = 0.f;
    for (int c = threadIdx.x; c < hidden; c += LANE_THREADS) {
        float sum = 0.f;
        for (int l = 0; l < count; ++l) {
            const float value = lanes[l * lane_stride + s * hidden + c];
            sum = l == 0 ? (read ? read[0] * value : value) : (read ? fmaf(read[l], value, sum) : sum + value);
        }
        staged[c] = sum;
        square = fmaf(sum, sum, square);
    }
    float inv = 1.f;
    if (weight) inv = 1.0f / sqrtf(block_sum<LANE_THREADS>(square, scratch) / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += LANE_THREADS) {
        const float value = weight ? staged[c] * inv * to_float(weight[c]) : staged[c];
        y[(long long)r * hidden + c] = from_float<TY>(value);
    }
}

// A thread per element of a lane. `source` may be `target` (in place: a thread reads every lane's element
// before it writes any) or one matrix that stands for every lane (source_stride 0).
template <typename TY>
__global__ void lanes_mix_kernel(const float* source, long long source_stride, float* target, long long target_stride,
                                 int count, const float* __restrict__ mix, const float* __restrict__ write,
                                 const TY* __restrict__ y, long long total) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    float old[MAX_LANES];
#pragma unroll
    for (int l = 0; l < MAX_LANES; ++l)
        if (l < count) old[l] = source[l * source_stride + index];
    const float delta = to_float(y[index]);
#pragma unroll
    for (int t = 0; t < MAX_LANES; ++t) {
        if (t >= count) break;
        float sum = 0.f;
#pragma unroll
        for (int l = 0; l < MAX_LANES; ++l)
            if (l < count) sum = l == 0 ? mix[t] * old[0] : fmaf(mix[l * count + t], old[l], sum);
        target[t * target_stride + index] = fmaf(write[t], delta, sum);
    }
}

// Four consecutive elements as 32-bit values (the address is aligned to four elements).
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = raw;
}

// The same as lanes_rmsnorm_kernel for widths that are multiples of four and aligned rows: four elements a thread and
// step, the loads of all lanes in flight together. The sums are formed in the same order.
template <typename TW, typename TY>
__global__ void __launch_bounds__(LANE_THREADS)
lanes_rmsnorm_x4_kernel(const float* __restrict__ lanes, long long lane_stride, int count, const float* __restrict__ read,
                        const TW* __restrict__ weight, TY* __restrict__ y, const int* __restrict__ row_index, int hidden,
                        float eps) {
    extern __shared__ __align__(16) float staged[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float square = 0.f;
    for (int c = 4 * threadIdx.x; c < hidden; c += 4 * LANE_THREADS) {
        float sum[4];
        for (int l = 0; l < count; ++l) {
            float value[4];
            load4(lanes + l * lane_stride + s * hidden + c, value);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                sum[i] = l == 0 ? (read ? read[0] * value[i] : value[i])
                                : (read ? fmaf(read[l], value[i], sum[i]) : sum[i] + value[i]);
        }
        store4(staged + c, sum);
#pragma unroll
        for (int i = 0; i < 4; ++i) square = fmaf(sum[i], sum[i], square);
    }
    float inv = 1.f;
    if (weight) inv = 1.0f / sqrtf(block_sum<LANE_THREADS>(square, scratch) / (float)hidden + eps);
    for (int c = 4 * threadIdx.x; c < hidden; c += 4 * LANE_THREADS) {
        float value[4], w[4];
        load4(staged + c, value);
        if (weight) {
            load4(weight + c, w);
#pragma unroll
            for (int i = 0; i < 4; ++i) value[i] = value[i] * inv * w[i];
        }
        store4(y + (long long)r * hidden + c, value);
    }
}

// lanes_mix_kernel, four elements a thread.
template <typename TY>
__global__ void lanes_mix_x4_kernel(const float* source, long long source_stride, float* target, long long target_stride,
                                    int count, const float* __restrict__ mix, const float* __restrict__ write,
                                    const TY* __restrict__ y, long long groups) {
    const long long index = 4 * ((long long)blockIdx.x * blockDim.x + threadIdx.x);
    if (index >= 4 * groups) return;
    float old[MAX_LANES][4], delta[4];
#pragma unroll
    for (int l = 0; l < MAX_LANES; ++l)
        if (l < count) load4(source + l * source_stride + index, old[l]);
    load4(y + index, delta);
#pragma unroll
    for (int t = 0; t < MAX_LANES; ++t) {
        if (t >= count) break;
        float sum[4];
#pragma unroll
        for (int l = 0; l < MAX_LANES; ++l)
            if (l < count) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    sum[i] = l == 0 ? mix[t] * old[0][i] : fmaf(mix[l * count + t], old[l][i], sum[i]);
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) sum[i] = fmaf(write[t], delta[i], sum[i]);
        store4(target + t * target_stride + index, sum);
    }
}

// lanes_mix and lanes_rmsnorm in one pass (widths that are multiples of four): a block per output row forms the new
// lanes from the old ones and the sublayer's result y, writes them (unless only picked rows are wanted: the stream is
// then left as it is), and reads them at once as the next sublayer's weighted sum, with its norm. Every sum is formed in
// the order of the two kernels it replaces: the same bits.
template <typename TD, typename TW, typename TY>
__global__ void __launch_bounds__(LANE_THREADS)
lanes_mix_rmsnorm_kernel(const float* source, long long source_stride, float* target, long long target_stride, int count,
                         const float* __restrict__ mix, const float* __restrict__ write, const TD* __restrict__ delta,
                         const float* __restrict__ read, const TW* __restrict__ weight, TY* __restrict__ y,
                         const int* __restrict__ row_index, int hidden, float eps) {
    extern __shared__ __align__(16) float staged[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float square = 0.f;
    for (int c = 4 * threadIdx.x; c < hidden; c += 4 * LANE_THREADS) {
        float old[MAX_LANES][4], d[4], sum[4];
#pragma unroll
        for (int l = 0; l < MAX_LANES; ++l)
            if (l < count) load4(source + l * source_stride + s * hidden + c, old[l]);
        load4(delta + s * hidden + c, d);
#pragma unroll
        for (int t = 0; t < MAX_LANES; ++t) {
            if (t >= count) break;
            float fresh[4];
#pragma unroll
            for (int l = 0; l < MAX_LANES; ++l)
                if (l < count) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        fresh[i] = l == 0 ? mix[t] * old[0][i] : fmaf(mix[l * count + t], old[l][i], fresh[i]);
                }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                fresh[i] = fmaf(write[t], d[i], fresh[i]);
                sum[i] = t == 0 ? (read ? read[0] * fresh[i] : fresh[i])
                                : (read ? fmaf(read[t], fresh[i], sum[i]) : sum[i] + fresh[i]);
            }
            if (!row_index) store4(target + t * target_stride + s * hidden + c, fresh);
        }
        store4(staged + c, sum);
#pragma unroll
        for (int i = 0; i < 4; ++i) square = fmaf(sum[i], sum[i], square);
    }
    const float inv = 1.0f / sqrtf(block_sum<LANE_THREADS>(square, scratch) / (float)hidden + eps);
    for (int c = 4 * threadIdx.x; c < hidden; c += 4 * LANE_THREADS) {
        float value[4], w[4];
        load4(staged + c, value);
        load4(weight + c, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) value[i] = value[i] * inv * w[i];
        store4(y + (long long)r * hidden + c, value);
    }
}

// One block per row: both rows staged, their mean squares, then the weighted sum of the two normalised rows.
template <typename T, typename TY>
__global__ void __launch_bounds__(LANE_THREADS)
normed_pair_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                       const float* __restrict__ wb, float ca, float cb, TY* __restrict__ out, int hidden, float eps) {
    extern __shared__ float staged[];
    __shared__ float scratch[32];
    const long long r = blockIdx.x;
    float* first = staged;
    float* second = staged + hidden;
    float square_a = 0.f, square_b = 0.f;
    for (int c = threadIdx.x; c < hidden; c += LANE_THREADS) {
        const float x = to_float(a[r * hidden + c]), z = to_float(b[r * hidden + c]);
        first[c] = x;
        second[c] = z;
        square_a = fmaf(x, x, square_a);
        square_b = fmaf(z, z, square_b);
    }
    const float inv_a = 1.0f / sqrtf(block_sum<LANE_THREADS>(square_a, scratch) / (float)hidden + eps);
    const float inv_b = 1.0f / sqrtf(block_sum<LANE_THREADS>(square_b, scratch) / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += LANE_THREADS)
        out[r * hidden + c] = from_float<TY>(ca * (first[c] * inv_a * wa[c]) + cb * (second[c] * inv_b * wb[c]));
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, long long ldx, const T* __restrict__ gate, long long ldg,
                                    int width, long long total) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / width;
    const int c = (int)(index - row * width);
    const float g = to_float(gate[row * ldg + c]);
    x[row * ldx + c] = from_float<T>(to_float(x[row * ldx + c]) / (1.0f + expf(-g)));
}

template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ z, T* __restrict__ out, long long total) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const float value = fmaxf(to_float(z[index]), 0.f);
    out[index] = from_float<T>(value * value);
}

// eight bfloat16 values a thread (16-byte pieces)
__global__ void relu_squared_bf16x8_kernel(const bf16* __restrict__ z, bf16* __restrict__ out, long long groups) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= groups) return;
    const uint4 raw = reinterpret_cast<const uint4*>(z)[index];
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 packed;
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 two = __bfloat1622float2(pairs[i]);
        const float x = fmaxf(two.x, 0.f), w = fmaxf(two.y, 0.f);
        result[i] = __floats2bfloat162_rn(x * x, w * w);
    }
    reinterpret_cast<uint4*>(out)[index] = packed;
}

template <typename TW>
int lanes_rmsnorm_out(const float* lanes, long long lane_stride, int count, const float* read, const TW* weight, void* y,
                      int y_dtype, const int* row_index, int rows, int hidden, float eps, cudaStream_t stream) {
    const size_t shared = (size_t)hidden * sizeof(float);
    const bool x4 = hidden % 4 == 0 && lane_stride % 4 == 0 && !((uintptr_t)lanes & 15) && !((uintptr_t)weight & 15) &&
                    !((uintptr_t)y & 15);
    if (y_dtype == KIDI_F32) {
        auto kernel = x4 ? lanes_rmsnorm_x4_kernel<TW, float> : lanes_rmsnorm_kernel<TW, float>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, lanes, lane_stride, count, read, weight, (float*)y,
                           row_index, hidden, eps);
    }
    if (y_dtype == KIDI_BF16) {
        auto kernel = x4 ? lanes_rmsnorm_x4_kernel<TW, bf16> : lanes_rmsnorm_kernel<TW, bf16>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, lanes, lane_stride, count, read, weight, (bf16*)y,
                           row_index, hidden, eps);
    }
    return KIDI_REFUSED_DTYPE;
}

template <typename T>
int normed_pair_sum_out(const T* a, const T* b, const float* wa, const float* wb, float ca, float cb, void* out,
                        int out_dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    const size_t shared = (size_t)2 * hidden * sizeof(float);
    if (out_dtype == KIDI_F32) {
        auto kernel = normed_pair_sum_kernel<T, float>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, a, b, wa, wb, ca, cb, (float*)out, hidden, eps);
    }
    if (out_dtype == KIDI_BF16) {
        auto kernel = normed_pair_sum_kernel<T, bf16>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, a, b, wa, wb, ca, cb, (bf16*)out, hidden, eps);
    }
    return KIDI_REFUSED_DTYPE;
}

}  // namespace

KIDI_API int kidi_lanes_rmsnorm(const float* lanes, long long lane_stride, int count, const float* read,
                                const void* weight, int weight_dtype, void* y, int y_dtype, const int* row_index,
                                int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (count <= 0 || count > MAX_LANES || hidden <= 0 || (size_t)hidden * sizeof(float) > 200 * 1024)
        return KIDI_REFUSED_SIZE;
    if (!weight || weight_dtype == KIDI_F32)
        return lanes_rmsnorm_out<float>(lanes, lane_stride, count, read, (const float*)weight, y, y_dtype, row_index,
                                        rows, hidden, eps, stream);
    if (weight_dtype == KIDI_BF16)
        return lanes_rmsnorm_out<bf16>(lanes, lane_stride, count, read, (const bf16*)weight, y, y_dtype, row_index, rows,
                                       hidden, eps, stream);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_lanes_mix(const float* source, long long source_stride, float* target, long long target_stride,
                            int count, const float* mix, const float* write, const void* y, int y_dtype,
                            long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (count <= 0 || count > MAX_LANES) return KIDI_REFUSED_SIZE;
    if (total % 4 == 0 && source_stride % 4 == 0 && target_stride % 4 == 0 && !((uintptr_t)source & 15) &&
        !((uintptr_t)target & 15) && !((uintptr_t)y & 15)) {
        const long long groups = total / 4;
        const unsigned vector_blocks = (unsigned)((groups + 255) / 256);
        if (y_dtype == KIDI_F32)
            return kidi_launch(lanes_mix_x4_kernel<float>, vector_blocks, 256, 0, stream, source, source_stride, target,
                               target_stride, count, mix, write, (const float*)y, groups);
        if (y_dtype == KIDI_BF16)
            return kidi_launch(lanes_mix_x4_kernel<bf16>, vector_blocks, 256, 0, stream, source, source_stride, target,
                               target_stride, count, mix, write, (const bf16*)y, groups);
        return KIDI_REFUSED_DTYPE;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (y_dtype == KIDI_F32)
        return kidi_launch(lanes_mix_kernel<float>, blocks, 256, 0, stream, source, source_stride, target, target_stride,
                           count, mix, write, (const float*)y, total);
    if (y_dtype == KIDI_BF16)
        return kidi_launch(lanes_mix_kernel<bf16>, blocks, 256, 0, stream, source, source_stride, target, target_stride,
                           count, mix, write, (const bf16*)y, total);
    return KIDI_REFUSED_DTYPE;
}

namespace {
template <typename TD, typename TW>
int lanes_mix_rmsnorm_out(const float* source, long long source_stride, float* target, long long target_stride, int count,
                          const float* mix, const float* write, const TD* delta, const float* read, const TW* weight,
                          void* y, int y_dtype, const int* row_index, int rows, int hidden, float eps, cudaStream_t stream) {
    const size_t shared = (size_t)hidden * sizeof(float);
    if (y_dtype == KIDI_F32) {
        auto kernel = lanes_mix_rmsnorm_kernel<TD, TW, float>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, source, source_stride, target, target_stride, count,
                           mix, write, delta, read, weight, (float*)y, row_index, hidden, eps);
    }
    if (y_dtype == KIDI_BF16) {
        auto kernel = lanes_mix_rmsnorm_kernel<TD, TW, bf16>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, rows, LANE_THREADS, shared, stream, source, source_stride, target, target_stride, count,
                           mix, write, delta, read, weight, (bf16*)y, row_index, hidden, eps);
    }
    return KIDI_REFUSED_DTYPE;
}

template <typename TD>
int lanes_mix_rmsnorm_weight(const float* source, long long source_stride, float* target, long long target_stride,
                             int count, const float* mix, const float* write, const TD* delta, const float* read,
                             const void* weight, int weight_dtype, void* y, int y_dtype, const int* row_index, int rows,
                             int hidden, float eps, cudaStream_t stream) {
    if (weight_dtype == KIDI_F32)
        return lanes_mix_rmsnorm_out<TD, float>(source, source_stride, target, target_stride, count, mix, write, delta,
                                                read, (const float*)weight, y, y_dtype, row_index, rows, hidden, eps, stream);
    if (weight_dtype == KIDI_BF16)
        return lanes_mix_rmsnorm_out<TD, bf16>(source, source_stride, target, target_stride, count, mix, write, delta, read,
                                               (const bf16*)weight, y, y_dtype, row_index, rows, hidden, eps, stream);
    return KIDI_REFUSED_DTYPE;
}
}  // namespace

// Refuses (KIDI_REFUSED_SIZE) what the four-element form does not take; the caller then runs the two kernels.
KIDI_API int kidi_lanes_mix_rmsnorm(const float* source, long long source_stride, float* target, long long target_stride,
                                    int count, const float* mix, const float* write, const void* delta, int delta_dtype,
                                    const float* read, const void* weight, int weight_dtype, void* y, int y_dtype,
                                    const int* row_index, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (count <= 0 || count > MAX_LANES || hidden <= 0 || hidden % 4 || (size_t)hidden * sizeof(float) > 200 * 1024 ||
        source_stride % 4 || target_stride % 4 || !weight || ((uintptr_t)source & 15) || ((uintptr_t)target & 15) ||
        ((uintptr_t)delta & 15) || ((uintptr_t)weight & 15) || ((uintptr_t)y & 15))
        return KIDI_REFUSED_SIZE;
    if (delta_dtype == KIDI_F32)
        return lanes_mix_rmsnorm_weight<float>(source, source_stride, target, target_stride, count, mix, write,
                                               (const float*)delta, read, weight, weight_dtype, y, y_dtype, row_index, rows,
                                               hidden, eps, stream);
    if (delta_dtype == KIDI_BF16)
        return lanes_mix_rmsnorm_weight<bf16>(source, source_stride, target, target_stride, count, mix, write,
                                              (const bf16*)delta, read, weight, weight_dtype, y, y_dtype, row_index, rows,
                                              hidden, eps, stream);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_normed_pair_sum(const void* a, const void* b, int dtype, const float* wa, const float* wb, float ca,
                                  float cb, void* out, int out_dtype, int rows, int hidden, float eps,
                                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (size_t)2 * hidden * sizeof(float) > 200 * 1024) return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32)
        return normed_pair_sum_out<float>((const float*)a, (const float*)b, wa, wb, ca, cb, out, out_dtype, rows, hidden,
                                          eps, stream);
    if (dtype == KIDI_BF16)
        return normed_pair_sum_out<bf16>((const bf16*)a, (const bf16*)b, wa, wb, ca, cb, out, out_dtype, rows, hidden,
                                         eps, stream);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_sigmoid_gate(void* x, long long ldx, const void* gate, long long ldg, int dtype, int rows, int width,
                               cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32)
        return kidi_launch(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, (float*)x, ldx, (const float*)gate, ldg,
                           width, total);
    if (dtype == KIDI_BF16)
        return kidi_launch(sigmoid_gate_kernel<bf16>, blocks, 256, 0, stream, (bf16*)x, ldx, (const bf16*)gate, ldg, width,
                           total);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_relu_squared(const void* z, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (dtype == KIDI_BF16 && total % 8 == 0 && !((uintptr_t)z & 15) && !((uintptr_t)out & 15)) {
        const long long groups = total / 8;
        return kidi_launch(relu_squared_bf16x8_kernel, (unsigned)((groups + 255) / 256), 256, 0, stream, (const bf16*)z,
                           (bf16*)out, groups);
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32)
        return kidi_launch(relu_squared_kernel<float>, blocks, 256, 0, stream, (const float*)z, (float*)out, total);
    if (dtype == KIDI_BF16)
        return kidi_launch(relu_squared_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)z, (bf16*)out, total);
    return KIDI_REFUSED_DTYPE;
}
