// A feed-forward made of many small experts, of which each token uses a few.
//
//   z = W_router h (32-bit), s = score(z), a sigmoid of each logit or a softmax over all of them; the `top`
//   experts with the largest scores are taken (ties: the lower index) with weights w = s (optionally divided
//   by their sum plus a small number). With groups, the experts form equal runs of neighbours, a group's
//   score is its largest, and only experts of the `keep` best groups (ties: the lower index) can be taken;
//   y = sum over the chosen experts of  scale_out * W_down[e] (act(W_gate[e] x) * (W_up[e] x)),
//   x = scale_in * h, where the weight w is scale_in (a weight on the expert's input) or scale_out
//   (on its output) and the other is 1. act is SiLU. An expert without a gate is W_down[e] gelu(W_up[e] x)
//   with the exact gelu, 0.5 z (1 + erf(z / sqrt 2)).
//
// A (row, choice) pair is a "slot": slot = row * top + choice.
//
// Kernels:
//  * choose: the router's product, the scores, the top choices and their weights, a block a row;
//  * slots, gate and up: for few rows, and for every row count of the 32-bit engine: a warp per
//    (slot, feature) reads the chosen expert's two weight rows once and applies the activation; the
//    input weight is applied to the two products in 32-bit (W (w h) = w (W h));
//  * slots, down: a warp per (row, feature) sums its choices' products in the order of the choices;
//  * gather / combine: for many rows the slots are sorted by expert on the host, their scaled input
//    rows gathered, each expert's rows run through the ordinary products, and the results summed per
//    row in the order of the choices.
// Nothing here depends on which other rows share the step: a row's result is the same alone and in
// a batch.
#include "common.cuh"

// ---------------------------------------------------------------- choose
// One row of weights against one row of x, a warp's share; the caller sums over the warp.
template <typename T, typename TW>
__device__ __forceinline__ float dot1(const TW* __restrict__ w, const T* __restrict__ x, int K, int lane) {
    float a = 0.f;
    for (int k = lane; k < K; k += 32) a = fmaf(to_float(w[k]), to_float(x[k]), a);
    return a;
}
template <>
__device__ __forceinline__ float dot1<bf16, bf16>(const bf16* __restrict__ w, const bf16* __restrict__ x, int K, int lane) {
    float a = 0.f;
    if ((K & 7) || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) {
        for (int k = lane; k < K; k += 32) a = fmaf(to_float(w[k]), to_float(x[k]), a);
        return a;
    }
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 rw = *reinterpret_cast<const uint4*>(w + k), rx = *reinterpret_cast<const uint4*>(x + k);
        const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&rw);
        const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&rx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fw = __bfloat1622float2(pw[i]), fx = __bfloat1622float2(px[i]);
            a = fmaf(fw.x, fx.x, a);
            a = fmaf(fw.y, fx.y, a);
        }
    }
    return a;
}

// A block a row: its sixteen warps share the experts (a warp a router row at a time, 32-bit sums in an order
// that depends on the width only), then the first warp takes the `top` largest scores, one after the other.
template <typename T, typename TW>
__global__ void __launch_bounds__(512) route_kernel(const T* __restrict__ x, const TW* __restrict__ router,
                                                    int* __restrict__ chosen, float* __restrict__ weight, int hidden,
                                                    int experts, int top, int renormalise, int softmax, int groups,
                                                    int keep, float renormalise_eps) {
    extern __shared__ float score[];       // [experts] scores, then [experts] what may still be chosen
    float* open = score + experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = blockIdx.x;
    for (int e = warp; e < experts; e += 16) {
        const float z = warp_sum(dot1<T, TW>(router + (long long)e * hidden, x + row * hidden, hidden, lane));
        if (lane == 0) score[e] = softmax ? z : 1.0f / (1.0f + expf(-z));
    }
    __syncthreads();
    if (warp) return;
    if (softmax) {                         // over all experts, the sum in lane order and then across the lanes
        float most = -INFINITY;
        for (int e = lane; e < experts; e += 32) most = fmaxf(most, score[e]);
        most = warp_max(most);
        float sum = 0.f;
        for (int e = lane; e < experts; e += 32) sum += expf(score[e] - most);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - most) / sum;
        __syncwarp();
    }
    for (int e = lane; e < experts; e += 32) open[e] = score[e];
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // The best `keep` groups stay open: one after the other the group with the largest best score is marked,
        // then every expert of an unmarked group is closed. A lane looks after groups lane, lane + 32, ...
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, score[e]);
            // a group's best score is kept in its first expert's `open` entry while the groups are ranked
            open[g * per] = best;
        }
        __syncwarp();
        unsigned long long kept_low = 0ull;      // groups kept by this lane, bit j for group lane + 32 j
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane, j = 0; g < groups; g += 32, ++j) {
                if (kept_low >> j & 1ull) continue;
                const float s = open[g * per];
                if (s > best) { best = s; at = g; }
            }
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, offset);
                const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
                if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
            }
            if (at == 0x7fffffff) break;
            if ((at & 31) == lane) kept_low |= 1ull << (at >> 5);
        }
        __syncwarp();
        for (int g = lane, j = 0; g < groups; g += 32, ++j) {
            const bool kept = kept_low >> j & 1ull;
            for (int e = g * per; e < (g + 1) * per; ++e) open[e] = kept ? score[e] : -INFINITY;
        }
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float s = open[e];
            if (s > best) { best = s; at = e; }          // ascending e: the first of equals stays
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
            if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
        }
        if (at == 0x7fffffff) { at = k; best = score[k]; }   // every score left is a NaN or closed
        if (lane == 0) {
            chosen[row * top + k] = at;
            weight[row * top + k] = best;
            open[at] = -INFINITY;
        }
        total += best;
        __syncwarp();
    }
    if (renormalise && lane < top) weight[row * top + lane] /= total + renormalise_eps;
}

KIDI_API int kidi_route(const void* x, int dtype, const void* router, int weight_dtype, int* chosen, float* weight,
                        int rows, int hidden, int experts, int top, int renormalise, int softmax, int groups, int keep,
                        float renormalise_eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (experts <= 0 || experts > 1024 || top <= 0 || top > experts || top > 32) return KIDI_REFUSED_SIZE;
    if (groups < 1 || experts % groups || keep < 1 || keep > groups || groups > 2048 ||
        (long long)keep * (experts / groups) < top)
        return KIDI_REFUSED_SIZE;
    const size_t shared = (size_t)experts * 2 * sizeof(float);
#define KIDI_CASE(D, T, W, TW)                                                                                        \
    if (dtype == D && weight_dtype == W)                                                                              \
        return kidi_launch(route_kernel<T, TW>, (unsigned)rows, 512, shared, stream, (const T*)x, (const TW*)router,  \
                           chosen, weight, hidden, experts, top, renormalise, softmax, groups, keep, renormalise_eps);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// ------------------------------------------------------------------ dots
// Two rows of weights against one row of x, a warp's share; the caller sums over the warp.
template <typename T>
__device__ __forceinline__ void dot2(const T* __restrict__ wa, const T* __restrict__ wb, const T* __restrict__ x, int K,
                                     int lane, float& a, float& b) {
    for (int k = lane; k < K; k += 32) {
        const float v = to_float(x[k]);
        a = fmaf(to_float(wa[k]), v, a);
        b = fmaf(to_float(wb[k]), v, b);
    }
}
template <>
__device__ __forceinline__ void dot2<bf16>(const bf16* __restrict__ wa, const bf16* __restrict__ wb,
                                           const bf16* __restrict__ x, int K, int lane, float& a, float& b) {
    if ((K & 7) || ((uintptr_t)wa & 15) || ((uintptr_t)wb & 15) || ((uintptr_t)x & 15)) {
        for (int k = lane; k < K; k += 32) {
            const float v = to_float(x[k]);
            a = fmaf(to_float(wa[k]), v, a);
            b = fmaf(to_float(wb[k]), v, b);
        }
        return;
    }
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 ra = *reinterpret_cast<const uint4*>(wa + k), rb = *reinterpret_cast<const uint4*>(wb + k);
        const uint4 rx = *reinterpret_cast<const uint4*>(x + k);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
        const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&rx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]), fx = __bfloat1622float2(px[i]);
            a = fmaf(fa.x, fx.x, a); a = fmaf(fa.y, fx.y, a);
            b = fmaf(fb.x, fx.x, b); b = fmaf(fb.y, fx.y, b);
        }
    }
}

// ----------------------------------------------------- slots: gate and up
// gate_up [experts, 2 * inter, hidden] (gate rows, then up rows); mid [rows * top, inter].
template <typename T, typename TW>
__global__ void __launch_bounds__(128) expert_gate_up_kernel(const T* __restrict__ x, const TW* __restrict__ gate_up,
                                                             const int* __restrict__ chosen, const float* __restrict__ weight,
                                                             T* __restrict__ mid, long long slots, int top, int hidden,
                                                             int inter, int weight_on_input, int gated) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= slots * inter) return;
    const long long slot = item / inter;
    const int n = (int)(item - slot * inter);
    const int expert = chosen[slot];
    const TW* base = gate_up + (long long)expert * (gated ? 2 : 1) * inter * hidden;
    const T* row = x + (slot / top) * hidden;
    const long long second = gated ? inter + n : n;     // without a gate there is one row: both sums are the same
    float g = 0.f, u = 0.f;
    if constexpr (sizeof(T) == sizeof(TW)) dot2<T>((const T*)base + (long long)n * hidden,
                                                   (const T*)base + second * hidden, row, hidden, lane, g, u);
    else
        for (int k = lane; k < hidden; k += 32) {
            const float v = to_float(row[k]);
            g = fmaf(to_float(base[(long long)n * hidden + k]), v, g);
            u = fmaf(to_float(base[second * hidden + k]), v, u);
        }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
        const float w = weight_on_input ? weight[slot] : 1.f;
        g *= w;
        u *= w;
        mid[slot * inter + n] = from_float<T>(gated ? g / (1.0f + expf(-g)) * u
                                                    : 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)));
    }
}

// ---------------------------------------------------------- slots: down
// down [experts, hidden, inter]; out [rows, hidden] = sum over a row's choices, in their order (plus `addend`
// [rows, hidden], if given: the result of an expert that every row passes).
template <typename T, typename TW>
__global__ void __launch_bounds__(128) expert_down_kernel(const T* __restrict__ mid, const TW* __restrict__ down,
                                                          const int* __restrict__ chosen, const float* __restrict__ weight,
                                                          T* __restrict__ out, long long rows, int top, int hidden, int inter,
                                                          int weight_on_input, const T* __restrict__ addend) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= rows * hidden) return;
    const long long row = item / hidden;
    const int n = (int)(item - row * hidden);
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const long long slot = row * top + k;
        const TW* w = down + ((long long)chosen[slot] * hidden + n) * inter;
        const T* m = mid + slot * inter;
        float a = 0.f, unused = 0.f;
        if constexpr (sizeof(T) == sizeof(TW)) dot2<T>((const T*)w, (const T*)w, m, inter, lane, a, unused);
        else
            for (int i = lane; i < inter; i += 32) a = fmaf(to_float(w[i]), to_float(m[i]), a);
        a = warp_sum(a);
        total += weight_on_input ? a : a * weight[slot];
    }
    if (lane == 0) out[row * hidden + n] = from_float<T>(addend ? total + to_float(addend[row * hidden + n]) : total);
}

KIDI_API int kidi_expert_slots(const void* x, int dtype, const void* gate_up, const void* down, int weight_dtype,
                               const int* chosen, const float* weight, void* mid, void* out, int rows, int top,
                               int hidden, int inter, int weight_on_input, int gated, const void* addend,
                               cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long slots = (long long)rows * top;
    const long long first = slots * inter, second = (long long)rows * hidden;
    if (first >= (1LL << 33) || second >= (1LL << 33)) return KIDI_REFUSED_SIZE;
#define KIDI_CASE(D, T, W, TW)                                                                                     \
    if (dtype == D && weight_dtype == W) {                                                                         \
        int status = kidi_launch(expert_gate_up_kernel<T, TW>, (unsigned)((first + 3) / 4), 128, 0, stream,       \
                                 (const T*)x, (const TW*)gate_up, chosen, weight, (T*)mid, slots, top, hidden,     \
                                 inter, weight_on_input, gated);                                                   \
        if (status) return status;                                                                                 \
        return kidi_launch(expert_down_kernel<T, TW>, (unsigned)((second + 3) / 4), 128, 0, stream, (const T*)mid, \
                           (const TW*)down, chosen, weight, (T*)out, (long long)rows, top, hidden, inter,          \
                           weight_on_input, (const T*)addend);                                                     \
    }
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// ------------------------------------------------------ gather / combine
// gathered[i] = x[order[i] / top] * (weight[order[i]] or 1): the slots' input rows in the order of their experts
// (order[i] < 0: a row of zeros, where every expert's rows are padded to one count).
template <typename T>
__global__ void gather_slots_kernel(const T* __restrict__ x, const int* __restrict__ order, const float* __restrict__ weight,
                                    T* __restrict__ gathered, long long total, int top, int hidden, int weight_on_input) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long i = index / hidden;
    const int c = (int)(index - i * hidden);
    const int slot = order[i];
    if (slot < 0) { gathered[index] = from_float<T>(0.f); return; }          // a padding row
    const float w = weight_on_input ? weight[slot] : 1.f;
    gathered[index] = from_float<T>(to_float(x[(long long)(slot / top) * hidden + c]) * w);
}

// out[row] = sum over the row's choices k of y[place[row * top + k]] (* weight), in the order of the choices.
template <typename T>
__global__ void combine_slots_kernel(const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weight,
                                     T* __restrict__ out, long long total, int top, int hidden, int weight_on_input,
                                     const T* __restrict__ addend) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / hidden;
    const int c = (int)(index - row * hidden);
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        const long long slot = row * top + k;
        const float value = to_float(y[(long long)place[slot] * hidden + c]);
        sum += weight_on_input ? value : value * weight[slot];
    }
    if (addend) sum += to_float(addend[index]);
    out[index] = from_float<T>(sum);
}

// The same two for bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) a thread.
__global__ void gather_slots_bf16x8_kernel(const bf16* __restrict__ x, const int* __restrict__ order,
                                           const float* __restrict__ weight, bf16* __restrict__ gathered, long long groups,
                                           int top, int hidden, int weight_on_input) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= groups) return;
    const int per_row = hidden >> 3;
    const long long i = index / per_row;
    const int c = (int)(index - i * per_row) << 3;
    const int slot = order[i];
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);                                  // a padding row stays zero
    if (slot >= 0) raw = *reinterpret_cast<const uint4*>(x + (long long)(slot / top) * hidden + c);
    if (slot >= 0 && weight_on_input) {
        const float w = weight[slot];
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __bfloat1622float2(pairs[k]);
            pairs[k] = __floats2bfloat162_rn(v.x * w, v.y * w);
        }
    }
    *reinterpret_cast<uint4*>(gathered + i * hidden + c) = raw;
}

__global__ void combine_slots_bf16x8_kernel(const bf16* __restrict__ y, const int* __restrict__ place,
                                            const float* __restrict__ weight, bf16* __restrict__ out, long long groups,
                                            int top, int hidden, int weight_on_input, const bf16* __restrict__ addend) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= groups) return;
    const int per_row = hidden >> 3;
    const long long row = index / per_row;
    const int c = (int)(index - row * per_row) << 3;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
        const long long slot = row * top + k;
        const uint4 raw = *reinterpret_cast<const uint4*>(y + (long long)place[slot] * hidden + c);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float w = weight_on_input ? 1.f : weight[slot];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(pairs[j]);
            sum[2 * j] += weight_on_input ? v.x : v.x * w;
            sum[2 * j + 1] += weight_on_input ? v.y : v.y * w;
        }
    }
    if (addend) {
        const uint4 raw = *reinterpret_cast<const uint4*>(addend + row * hidden + c);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(pairs[j]);
            sum[2 * j] += v.x;
            sum[2 * j + 1] += v.y;
        }
    }
    uint4 result;
    __nv_bfloat162* packed = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int j = 0; j < 4; ++j) packed[j] = __floats2bfloat162_rn(sum[2 * j], sum[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + row * hidden + c) = result;
}

KIDI_API int kidi_gather_slots(const void* x, int dtype, const int* order, const float* weight, void* gathered, int slots,
                               int top, int hidden, int weight_on_input, cudaStream_t stream) {
    const long long total = (long long)slots * hidden;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(gather_slots_kernel<float>, blocks, 256, 0, stream, (const float*)x, order,
                                              weight, (float*)gathered, total, top, hidden, weight_on_input);
    if (dtype == KIDI_BF16 && !(hidden & 7) && !((uintptr_t)x & 15) && !((uintptr_t)gathered & 15))
        return kidi_launch(gather_slots_bf16x8_kernel, (unsigned)(((total >> 3) + 255) / 256), 256, 0, stream,
                           (const bf16*)x, order, weight, (bf16*)gathered, total >> 3, top, hidden, weight_on_input);
    if (dtype == KIDI_BF16) return kidi_launch(gather_slots_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)x, order,
                                               weight, (bf16*)gathered, total, top, hidden, weight_on_input);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_combine_slots(const void* y, int dtype, const int* place, const float* weight, void* out, int rows,
                                int top, int hidden, int weight_on_input, const void* addend, cudaStream_t stream) {
    const long long total = (long long)rows * hidden;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(combine_slots_kernel<float>, blocks, 256, 0, stream, (const float*)y, place,
                                              weight, (float*)out, total, top, hidden, weight_on_input, (const float*)addend);
    if (dtype == KIDI_BF16 && !(hidden & 7) && !((uintptr_t)y & 15) && !((uintptr_t)out & 15) && !((uintptr_t)addend & 15))
        return kidi_launch(combine_slots_bf16x8_kernel, (unsigned)(((total >> 3) + 255) / 256), 256, 0, stream,
                           (const bf16*)y, place, weight, (bf16*)out, total >> 3, top, hidden, weight_on_input,
                           (const bf16*)addend);
    if (dtype == KIDI_BF16) return kidi_launch(combine_slots_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)y, place,
                                               weight, (bf16*)out, total, top, hidden, weight_on_input, (const bf16*)addend);
    return KIDI_REFUSED_DTYPE;
}
