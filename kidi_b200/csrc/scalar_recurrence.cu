// Linear recurrences with a matrix state per head whose decay is one number per head and token:
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T            S: [dim, vdim] (+ one column whose "value" is 1, if asked for)
//     o_t = S_t^T q_t
//
// a_t (decay) and b_t (write strength) come computed, in 32-bit, from a gate kernel of the mixer that owns the
// recurrence; k, q (per head, or per group of heads) and v are columns of the mixer's projections. Two mixers
// are served, each with its gate kernel and its finishing kernel:
//
//  * a selective state-space mixer (Mamba-2): a = exp(-exp(A_log) dt), b = dt, dt = softplus(dt~ + bias), k = B,
//    q = C, v = x after a short causal convolution with SiLU; y = (o + D x) silu(z), RMS-normed in equal parts.
//  * a matrix memory with exponential gates (mLSTM): log gates i = cap tanh(i~ / cap), f = logsigmoid(cap
//    tanh(f~ / cap)), a running maximum m_t = max(f_t + m_(t-1), i_t) (m_0 = 0), a = exp(f + m_(t-1) - m_t),
//    b = exp(i - m_t); the extra state column is the normaliser n_t = a n_(t-1) + b k_t;
//    o <- o / (max(|n . q|, exp(-m_t)) + 1e-6), RMS-normed per head, times a weight, times sigmoid(g).
//
// The state lives in 32-bit floats per cache slot and is carried from token to token; gates, decays, the state,
// the read-out and the norms are 32-bit. The columns of a head's state are independent, so a block takes 32
// columns of one (sequence, head) and walks the sequence's rows of the step in order: a token's result depends on
// the sizes only, not on what else is in the step, nor on how the sequence was cut into steps.
#include "common.cuh"

struct ScalarRecurrenceArgs {
    const void* k;         // [rows, ldk]: key head j at j * dim
    long long ldk;
    const void* q;         // [rows, ldq]: query head j at j * dim
    long long ldq;
    const void* v;         // [rows, ldv]: value head h at h * vdim
    long long ldv;
    const float* coef;     // [rows, heads, coef_width]: a_t, b_t first
    float* state;          // [slots + 1, heads, dim, vdim + extra]
    float* out;            // [rows, heads * (vdim + extra)]: the read-out; column vdim of a head: n . q
    const int* row_seq;    // [rows] (-1: padding)
    const int* seq_slot;   // [seqs]
    const int* seq_row0;   // [seqs]
    const int* seq_len;    // [seqs]
    int seqs, heads, k_heads, q_heads, dim, vdim, extra, coef_width;
    float q_scale;         // q is multiplied by it
};

struct ShortConvArgs {
    const void* x;         // [rows, ldx]: the channels' inputs
    long long ldx;
    const float* weight;   // [channels, taps]: the last column multiplies the current token
    const float* bias;     // [channels] or null
    void* state;           // [slots + 1, taps - 1, channels]: a sequence's last taps - 1 inputs (zeros before its start)
    void* out;             // [rows, ldo]
    long long ldo;
    const int* row_seq;
    const int* row_pos;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_row0;
    const int* seq_len;
    int rows, seqs, channels, taps, silu;
};

namespace {

constexpr int THREADS = 256;
constexpr int MAX_CHUNK = 16;
constexpr int MAX_TAPS = 32;

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

// A load that stays where it is written and hands back the bits as they are, so that a chunk's loads are issued
// together, wait in registers while the chunk before is walked, and are converted only where they are used.
template <typename T> struct Raw;
template <> struct Raw<float> {
    typedef float type;
    static __device__ __forceinline__ type load(const float* pointer) {
        float value;
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(value) : "l"(pointer));
        return value;
    }
    static __device__ __forceinline__ float value(type bits) { return bits; }
};
template <> struct Raw<bf16> {
    typedef unsigned short type;
    static __device__ __forceinline__ type load(const bf16* pointer) {
        unsigned short bits;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(bits) : "l"(pointer));
        return bits;
    }
    static __device__ __forceinline__ float value(type bits) { return __uint_as_float((unsigned)bits << 16); }
};

// R: state rows a thread keeps in registers (dim <= GROUPS * R). Eight warps walk the block's 32 columns; warp g
// owns the state rows g R .. g R + R - 1. A ninth warp keeps, in the block of the head's first columns, the extra
// column (the state's rows dealt out over its lanes): its value is 1 for every token, so it needs no column of a
// block of its own. The keys (times b_t), queries (times q_scale), values and decays of a chunk of tokens are
// staged in shared memory a chunk ahead: their loads are issued before the chunk before is walked. COLUMNS: the
// state columns of a block, one a lane of a group of COLUMNS lanes (32: a warp; 16: half a warp, for steps that
// would otherwise leave most SMs without a block); GROUPS = 256 / COLUMNS groups share the state's rows.
template <typename T, int R, int COLUMNS>
__global__ void __launch_bounds__(THREADS + 32) scalar_recurrence_kernel(ScalarRecurrenceArgs a) {
    extern __shared__ __align__(16) float shared[];
    constexpr int GROUPS = THREADS / COLUMNS;
    constexpr int PADDED = GROUPS * R;
    constexpr int CHUNK = R >= 32 ? MAX_CHUNK / 2 : MAX_CHUNK;     // tokens staged at a time
    constexpr int ROW = 2 * PADDED + COLUMNS + 4;                  // keys | queries | values | decay (and padding)
    constexpr int KQ = (CHUNK * PADDED + THREADS - 1) / THREADS;
    constexpr int VV = (CHUNK * COLUMNS + THREADS - 1) / THREADS;
    constexpr int NR = (PADDED + 31) / 32;                         // rows of the extra column a lane keeps
    float* stage = shared;                                         // [2][CHUNK][ROW]
    float* partials = shared + 2 * CHUNK * ROW;                    // [2][CHUNK][GROUPS][COLUMNS]
    float* counted = partials + 2 * CHUNK * THREADS;               // [2][CHUNK][32]: the extra column's parts, a lane each
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.seq_row0[seq], count = a.seq_len[seq];
    if (count <= 0 || a.row_seq[row0] < 0) return;        // a padding sequence touches no state
    const int dim = a.dim, vdim = a.vdim, vcols = a.vdim + a.extra;
    const bool walker = threadIdx.x < THREADS;
    const bool counter = !walker && a.extra && blockIdx.z == 0;    // the warp that keeps the extra column
    const int lane = walker ? threadIdx.x % COLUMNS : threadIdx.x & 31, g = (threadIdx.x / COLUMNS) % GROUPS;
    const int column = blockIdx.z * COLUMNS + lane;
    const bool live = walker && column < vdim;
    const int k_head = head / (a.heads / a.k_heads), q_head = head / (a.heads / a.q_heads);
    float* state = a.state + ((long long)a.seq_slot[seq] * a.heads + head) * dim * vcols;
    float S[R], N[NR];
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        S[j] = live && d < dim ? state[(long long)d * vcols + column] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = lane + 32 * j;
        N[j] = counter && d < dim ? state[(long long)d * vcols + vdim] : 0.f;
    }
    typename Raw<T>::type raw_k[KQ], raw_q[KQ], raw_v[VV];
    float raw_write[KQ], raw_keep = 1.f;

    auto fetch = [&](int t0) {
        if (!walker) return;
        const int tokens = min(CHUNK, count - t0);
#pragma unroll
        for (int i = 0; i < KQ; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / PADDED, d = index - t * PADDED;
            raw_k[i] = raw_q[i] = 0;
            raw_write[i] = 0.f;
            if (t < tokens && d < dim) {
                const long long row = row0 + t0 + t;
                raw_k[i] = Raw<T>::load((const T*)a.k + row * a.ldk + (long long)k_head * dim + d);
                raw_q[i] = Raw<T>::load((const T*)a.q + row * a.ldq + (long long)q_head * dim + d);
                raw_write[i] = Raw<float>::load(a.coef + (row * a.heads + head) * a.coef_width + 1);
            }
        }
#pragma unroll
        for (int i = 0; i < VV; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / COLUMNS, c = index - t * COLUMNS;
            const int col = blockIdx.z * COLUMNS + c;
            raw_v[i] = 0;
            if (t < tokens && col < vdim)
                raw_v[i] = Raw<T>::load((const T*)a.v + (long long)(row0 + t0 + t) * a.ldv + (long long)head * vdim + col);
        }
        if (threadIdx.x < tokens)
            raw_keep = Raw<float>::load(a.coef + ((long long)(row0 + t0 + threadIdx.x) * a.heads + head) * a.coef_width);
    };
    auto put = [&](float* target) {
        if (!walker) return;
#pragma unroll
        for (int i = 0; i < KQ; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / PADDED, d = index - t * PADDED;
            if (index >= CHUNK * PADDED) continue;
            target[t * ROW + d] = raw_write[i] * Raw<T>::value(raw_k[i]);
            target[t * ROW + PADDED + d] = a.q_scale * Raw<T>::value(raw_q[i]);
        }
#pragma unroll
        for (int i = 0; i < VV; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / COLUMNS, c = index - t * COLUMNS;
            if (index < CHUNK * COLUMNS) target[t * ROW + 2 * PADDED + c] = Raw<T>::value(raw_v[i]);
        }
        if (threadIdx.x < CHUNK) target[threadIdx.x * ROW + 2 * PADDED + COLUMNS] = raw_keep;
    };

    fetch(0);
    put(stage);
    __syncthreads();
    int turn = 0;
    for (int t0 = 0; t0 < count; t0 += CHUNK, turn ^= 1) {
        const int tokens = min(CHUNK, count - t0);
        const bool more = t0 + CHUNK < count;
        if (more) fetch(t0 + CHUNK);                     // on their way while this chunk is walked
        const float* __restrict__ current = stage + turn * (CHUNK * ROW);
        float* __restrict__ partial = partials + turn * (CHUNK * GROUPS * COLUMNS);
        if (walker) {
#pragma unroll 2
            for (int t = 0; t < tokens; ++t) {       // (two tokens an iteration: the second one's loads go out early)
                const float* key = current + t * ROW + g * R;        // one address a warp: broadcasts
                const float* query = key + PADDED;
                const float keep = current[t * ROW + 2 * PADDED + COLUMNS];
                const float value = current[t * ROW + 2 * PADDED + lane];
                float sum = 0.f;
                if constexpr (R % 4 == 0) {
                    float sums[4] = {0.f, 0.f, 0.f, 0.f};            // four chains instead of one of R links
#pragma unroll
                    for (int j = 0; j < R; j += 4) {
                        const float4 k4 = *reinterpret_cast<const float4*>(key + j);
                        const float4 q4 = *reinterpret_cast<const float4*>(query + j);
                        const float kj[4] = {k4.x, k4.y, k4.z, k4.w}, qj[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float s = fmaf(keep, S[j + e], kj[e] * value);
                            S[j + e] = s;
                            sums[e] = fmaf(s, qj[e], sums[e]);
                        }
                    }
                    sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < R; ++j) {
                        const float s = fmaf(keep, S[j], key[j] * value);
                        S[j] = s;
                        sum = fmaf(s, query[j], sum);
                    }
                }
                partial[(t * GROUPS + g) * COLUMNS + lane] = sum;
            }
        } else if (counter) {
            for (int t = 0; t < tokens; ++t) {
                const float* key = current + t * ROW;
                const float keep = current[t * ROW + 2 * PADDED + COLUMNS];
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < NR; ++j) {
                    const int d = lane + 32 * j;
                    if (d < PADDED) {
                        N[j] = fmaf(keep, N[j], key[d]);
                        sum = fmaf(N[j], key[PADDED + d], sum);
                    }
                }
                counted[(turn * CHUNK + t) * 32 + lane] = sum;      // added up behind the barrier: no chain of
            }                                                        // shuffles a token holds the walkers up
        }
        if (more) put(stage + (turn ^ 1) * (CHUNK * ROW));
        __syncthreads();
        // (the stage and the partials written next are the other ones; these are free again behind the next barrier)
        for (int index = threadIdx.x; index < tokens * COLUMNS; index += THREADS + 32) {
            const int t = index / COLUMNS, c = index - t * COLUMNS;
            const int col = blockIdx.z * COLUMNS + c;
            if (col >= vdim) continue;
            float total = 0.f;
#pragma unroll
            for (int k = 0; k < GROUPS; ++k) total += partial[(t * GROUPS + k) * COLUMNS + c];
            a.out[((long long)(row0 + t0 + t) * a.heads + head) * vcols + col] = total;
        }
        if (a.extra && blockIdx.z == 0 && threadIdx.x < tokens) {      // n . q of the chunk's tokens, a thread each
            float total = 0.f;
#pragma unroll
            for (int l = 0; l < 32; ++l) total += counted[(turn * CHUNK + threadIdx.x) * 32 + l];
            a.out[((long long)(row0 + t0 + threadIdx.x) * a.heads + head) * vcols + vdim] = total;
        }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        if (live && d < dim) state[(long long)d * vcols + column] = S[j];
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = lane + 32 * j;
        if (counter && d < dim) state[(long long)d * vcols + vdim] = N[j];
    }
}

template <typename T, int R, int COLUMNS>
int launch_recurrence(const ScalarRecurrenceArgs& a, cudaStream_t stream) {
    constexpr int GROUPS = THREADS / COLUMNS;
    constexpr int PADDED = GROUPS * R;
    constexpr int CHUNK = R >= 32 ? MAX_CHUNK / 2 : MAX_CHUNK;
    const size_t shared = (size_t)2 * CHUNK * ((2 * PADDED + COLUMNS + 4) + GROUPS * COLUMNS + 32) * sizeof(float);
    auto kernel = scalar_recurrence_kernel<T, R, COLUMNS>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    dim3 grid(a.seqs, a.heads, (a.vdim + COLUMNS - 1) / COLUMNS);
    return kidi_launch(kernel, grid, THREADS + 32, shared, stream, a);
}

template <typename T, int COLUMNS>
int dispatch_rows(const ScalarRecurrenceArgs& a, cudaStream_t stream) {
    constexpr int GROUPS = THREADS / COLUMNS;
    const int rows = (a.dim + GROUPS - 1) / GROUPS;
    if (rows <= 1) return launch_recurrence<T, 1, COLUMNS>(a, stream);
    if (rows <= 2) return launch_recurrence<T, 2, COLUMNS>(a, stream);
    if (rows <= 4) return launch_recurrence<T, 4, COLUMNS>(a, stream);
    if (rows <= 8) return launch_recurrence<T, 8, COLUMNS>(a, stream);
    if (rows <= 16) return launch_recurrence<T, 16, COLUMNS>(a, stream);
    if (COLUMNS == 32 && rows <= 32) return launch_recurrence<T, 32, 32>(a, stream);
    return KIDI_REFUSED_SIZE;
}

template <typename T>
int dispatch_recurrence(const ScalarRecurrenceArgs& a, cudaStream_t stream) {
    // Few (sequence, head, 32 columns) blocks: half as many columns a block, so that SMs hold two blocks or more (a
    // block's walk is a chain of dependent steps: an SM needs several to fill its issue slots). The choice
    // depends on the step's sizes only through the number of sequences; a row's result does not depend on it
    // beyond the order in which the partial read-outs are added.
    const long long blocks = (long long)a.seqs * a.heads * ((a.vdim + 31) / 32);
    if (blocks < 2 * 148 && a.vdim > 16) return dispatch_rows<T, 16>(a, stream);
    return dispatch_rows<T, 32>(a, stream);
}

// ---------------------------------------------------------------- short causal convolution with carried inputs
// A thread per (row, channel): y = bias + sum_j w[c, j] x(position - (taps - 1) + j), inputs of earlier steps from
// the state, inputs before the sequence's start zero; then SiLU if asked. The sum is 32-bit.
template <typename T>
__global__ void short_conv_kernel(ShortConvArgs a) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (long long)a.rows * a.channels) return;
    const int row = (int)(index / a.channels), c = (int)(index - (long long)row * a.channels);
    const int seq = a.row_seq[row];
    if (seq < 0) return;
    const int position = a.row_pos[row], start = a.seq_start[seq], row0 = a.seq_row0[seq];
    const int reach = a.taps - 1;
    const T* state = (const T*)a.state + (long long)a.seq_slot[seq] * reach * a.channels;
    float sum = a.bias ? a.bias[c] : 0.f;
    for (int j = 0; j < a.taps; ++j) {
        const int p = position - reach + j;
        float x = 0.f;
        if (p >= start) x = to_float(((const T*)a.x)[(long long)(row0 + p - start) * a.ldx + c]);
        else if (p >= 0) x = to_float(state[(long long)(p - start + reach) * a.channels + c]);
        sum = fmaf(a.weight[(long long)c * a.taps + j], x, sum);
    }
    ((T*)a.out)[(long long)row * a.ldo + c] = from_float<T>(a.silu ? silu(sum) : sum);
}

// After the convolution: a sequence's last taps - 1 inputs, from the step's rows and (a step shorter than that) from
// what the state held. A thread per (sequence, channel) reads all it needs before it writes.
template <typename T>
__global__ void short_conv_state_kernel(ShortConvArgs a) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (long long)a.seqs * a.channels) return;
    const int seq = (int)(index / a.channels), c = (int)(index - (long long)seq * a.channels);
    const int row0 = a.seq_row0[seq], count = a.seq_len[seq];
    if (count <= 0 || a.row_seq[row0] < 0) return;
    const int reach = a.taps - 1;
    T* state = (T*)a.state + (long long)a.seq_slot[seq] * reach * a.channels;
    T kept[MAX_TAPS];
    for (int j = 0; j < reach; ++j) {
        const int back = reach - j;            // the input `back` tokens before the sequence's new end
        kept[j] = back <= count ? ((const T*)a.x)[(long long)(row0 + count - back) * a.ldx + c]
                                : state[(long long)(j + count) * a.channels + c];
    }
    for (int j = 0; j < reach; ++j) state[(long long)j * a.channels + c] = kept[j];
}

// One token a sequence (decoding): the output and the state's shift in one kernel, a thread a (sequence, channel); every
// earlier input comes from the state.
template <typename T>
__global__ void short_conv_step_kernel(ShortConvArgs a) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (long long)a.seqs * a.channels) return;
    const int seq = (int)(index / a.channels), c = (int)(index - (long long)seq * a.channels);
    const int row = a.seq_row0[seq];
    if (a.seq_len[seq] <= 0 || a.row_seq[row] < 0) return;
    const int reach = a.taps - 1;
    T* state = (T*)a.state + (long long)a.seq_slot[seq] * reach * a.channels;
    T kept[MAX_TAPS];
    float sum = a.bias ? a.bias[c] : 0.f;
    for (int j = 0; j < reach; ++j) {
        kept[j] = state[(long long)j * a.channels + c];
        sum = fmaf(a.weight[(long long)c * a.taps + j], to_float(kept[j]), sum);
    }
    const T x = ((const T*)a.x)[(long long)row * a.ldx + c];
    sum = fmaf(a.weight[(long long)c * a.taps + reach], to_float(x), sum);
    ((T*)a.out)[(long long)row * a.ldo + c] = from_float<T>(a.silu ? silu(sum) : sum);
    for (int j = 0; j + 1 < reach; ++j) state[(long long)j * a.channels + c] = kept[j + 1];
    if (reach > 0) state[(long long)(reach - 1) * a.channels + c] = x;
}

// ---------------------------------------------------------------- the state-space mixer's gates and finish
// coef[row, head] = (exp(-exp(A_log) dt), dt), dt = softplus(dt~ + bias) (no clamp).
template <typename T>
__global__ void state_space_gates_kernel(const T* __restrict__ dt, long long ld, const float* __restrict__ dt_bias,
                                         const float* __restrict__ a_log, float* __restrict__ coef, int rows, int heads) {
    const int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= rows * heads) return;
    const int row = index / heads, head = index - row * heads;
    const float raw = to_float(dt[(long long)row * ld + head]) + dt_bias[head];
    const float step = raw > 20.f ? raw : log1pf(expf(raw));
    coef[2 * index] = expf(-expf(a_log[head]) * step);
    coef[2 * index + 1] = step;
}

// A block per (row, part): y = (o + D x) silu(z) over the part's entries, divided by its root mean square, times
// the weight.
template <typename T>
__global__ void __launch_bounds__(THREADS)
state_space_finish_kernel(const float* __restrict__ read, const T* __restrict__ x, long long ldx, const T* __restrict__ z,
                          long long ldz, const float* __restrict__ skip, const float* __restrict__ weight,
                          T* __restrict__ out, long long ldo, int vdim, int part, float eps) {
    extern __shared__ float staged[];
    __shared__ float scratch[32];
    const long long row = blockIdx.x;
    const int begin = blockIdx.y * part;
    const int inner = gridDim.y * part;
    float square = 0.f;
    for (int i = threadIdx.x; i < part; i += THREADS) {
        const int c = begin + i;
        const float value = to_float(x[row * ldx + c]);
        const float y = (read[row * inner + c] + skip[c / vdim] * value) * silu(to_float(z[row * ldz + c]));
        staged[i] = y;
        square = fmaf(y, y, square);
    }
    const float inv = 1.0f / sqrtf(block_sum<THREADS>(square, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += THREADS)
        out[row * ldo + begin + i] = from_float<T>(staged[i] * inv * weight[begin + i]);
}

// ---------------------------------------------------------------- the matrix memory's gates and finish
// A warp per (sequence, head) walks the sequence's rows 32 at a time: each lane computes its token's log gates,
// the running maximum m_t = max(f_t + m_(t-1), i_t) is a scan of the maps m -> max(m + F, I) (composed:
// (F1, I1) then (F2, I2) = (F1 + F2, max(I1 + F2, I2))), and coef[row, head] = (exp(f + m_(t-1) - m_t),
// exp(i - m_t), exp(-m_t)). m is carried in `maximum` [slots + 1, heads].
template <typename T>
__global__ void matrix_memory_gates_kernel(const T* __restrict__ gates, long long ld, int offset_i, int offset_f,
                                           float cap, float* __restrict__ coef, float* __restrict__ maximum,
                                           const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
                                           const int* __restrict__ seq_row0, const int* __restrict__ seq_len, int seqs,
                                           int heads) {
    const int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (item >= seqs * heads) return;
    const int seq = item / heads, head = item - seq * heads;
    const int row0 = seq_row0[seq], count = seq_len[seq];
    if (count <= 0 || row_seq[row0] < 0) return;
    float* kept = maximum + (long long)seq_slot[seq] * heads + head;
    float m = *kept;
    for (int t0 = 0; t0 < count; t0 += 32) {
        const int t = t0 + lane;
        const bool live = t < count;
        float log_in = -INFINITY, log_keep = 0.f;      // beyond the end: the identity map
        if (live) {
            const T* row = gates + (long long)(row0 + t) * ld;
            log_in = cap * tanhf(to_float(row[offset_i + head]) / cap);
            const float bounded = cap * tanhf(to_float(row[offset_f + head]) / cap);
            log_keep = fminf(bounded, 0.f) - log1pf(expf(-fabsf(bounded)));      // log sigmoid
        }
        float F = log_keep, I = log_in;
#pragma unroll
        for (int step = 1; step < 32; step <<= 1) {
            const float F_before = __shfl_up_sync(0xffffffffu, F, step), I_before = __shfl_up_sync(0xffffffffu, I, step);
            if (lane >= step) {
                I = fmaxf(I_before + F, I);
                F = F_before + F;
            }
        }
        const float now = fmaxf(m + F, I);
        float before = __shfl_up_sync(0xffffffffu, now, 1);
        if (lane == 0) before = m;
        if (live) {
            float* target = coef + ((long long)(row0 + t) * heads + head) * 3;
            target[0] = expf(log_keep + before - now);
            target[1] = expf(log_in - now);
            target[2] = expf(-now);
        }
        m = __shfl_sync(0xffffffffu, now, min(31, count - t0 - 1));
    }
    if (lane == 0) *kept = m;
}

// A warp per (row, head): o / (max(|n . q|, exp(-m)) + 1e-6), divided by its root mean square over vdim, times the
// weight, times sigmoid(g).
template <typename T>
__global__ void matrix_memory_finish_kernel(const float* __restrict__ read, const float* __restrict__ coef,
                                            const float* __restrict__ weight, const T* __restrict__ gate, long long ldg,
                                            T* __restrict__ out, long long ldo, long long items, int heads, int vdim,
                                            float eps) {
    const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const long long row = item / heads;
    const int head = (int)(item - row * heads);
    const float* source = read + item * (vdim + 1);
    const float denominator = fmaxf(fabsf(source[vdim]), coef[item * 3 + 2]) + 1e-6f;
    float square = 0.f;
    for (int c = lane; c < vdim; c += 32) {
        const float value = source[c] / denominator;
        square = fmaf(value, value, square);
    }
    const float inv = 1.0f / sqrtf(warp_sum(square) / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
        const int column = head * vdim + c;
        const float g = to_float(gate[row * ldg + column]);
        out[row * ldo + column] = from_float<T>(source[c] / denominator * inv * weight[column] / (1.0f + expf(-g)));
    }
}

}  // namespace

KIDI_API int kidi_scalar_recurrence(const ScalarRecurrenceArgs* args, int dtype, cudaStream_t stream) {
    const ScalarRecurrenceArgs& a = *args;
    if (a.seqs <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.dim <= 0 || a.vdim <= 0 || a.extra < 0 || a.extra > 1 || a.k_heads <= 0 ||
        a.q_heads <= 0 || a.heads % a.k_heads || a.heads % a.q_heads || a.coef_width < 2 ||
        (a.vdim + 15) / 16 > 65535)
        return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return dispatch_recurrence<float>(a, stream);
    if (dtype == KIDI_BF16) return dispatch_recurrence<bf16>(a, stream);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_short_conv(const ShortConvArgs* args, int dtype, cudaStream_t stream) {
    const ShortConvArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.channels <= 0 || a.taps < 1 || a.taps > MAX_TAPS) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)(((long long)a.rows * a.channels + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(short_conv_kernel<float>, blocks, 256, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(short_conv_kernel<bf16>, blocks, 256, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_short_conv_state(const ShortConvArgs* args, int dtype, cudaStream_t stream) {
    const ShortConvArgs& a = *args;
    if (a.seqs <= 0 || a.taps <= 1) return 0;
    if (a.channels <= 0 || a.taps > MAX_TAPS) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)(((long long)a.seqs * a.channels + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(short_conv_state_kernel<float>, blocks, 256, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(short_conv_state_kernel<bf16>, blocks, 256, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_short_conv_step(const ShortConvArgs* args, int dtype, cudaStream_t stream) {
    const ShortConvArgs& a = *args;
    if (a.seqs <= 0) return 0;
    if (a.channels <= 0 || a.taps < 1 || a.taps > MAX_TAPS) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)(((long long)a.seqs * a.channels + 255) / 256);
    if (dtype == KIDI_F32) return kidi_launch(short_conv_step_kernel<float>, blocks, 256, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(short_conv_step_kernel<bf16>, blocks, 256, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_state_space_gates(const void* dt, long long ld, int dtype, const float* dt_bias, const float* a_log,
                                    float* coef, int rows, int heads, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || (long long)rows * heads > 0x7fffffff) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)((rows * heads + 255) / 256);
    if (dtype == KIDI_F32)
        return kidi_launch(state_space_gates_kernel<float>, blocks, 256, 0, stream, (const float*)dt, ld, dt_bias, a_log,
                           coef, rows, heads);
    if (dtype == KIDI_BF16)
        return kidi_launch(state_space_gates_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)dt, ld, dt_bias, a_log,
                           coef, rows, heads);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_state_space_finish(const float* read, const void* x, long long ldx, const void* z, long long ldz,
                                     int dtype, const float* skip, const float* weight, void* out, long long ldo,
                                     int rows, int heads, int vdim, int parts, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int inner = heads * vdim;
    if (heads <= 0 || vdim <= 0 || parts <= 0 || inner % parts || parts > 65535) return KIDI_REFUSED_SIZE;
    const int part = inner / parts;
    const size_t shared = (size_t)part * sizeof(float);
    if (shared > 200 * 1024) return KIDI_REFUSED_SIZE;
    dim3 grid(rows, parts);
    if (dtype == KIDI_F32) {
        auto kernel = state_space_finish_kernel<float>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, grid, THREADS, shared, stream, read, (const float*)x, ldx, (const float*)z, ldz, skip,
                           weight, (float*)out, ldo, vdim, part, eps);
    }
    if (dtype == KIDI_BF16) {
        auto kernel = state_space_finish_kernel<bf16>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        return kidi_launch(kernel, grid, THREADS, shared, stream, read, (const bf16*)x, ldx, (const bf16*)z, ldz, skip,
                           weight, (bf16*)out, ldo, vdim, part, eps);
    }
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_matrix_memory_gates(const void* gates, long long ld, int offset_i, int offset_f, int dtype, float cap,
                                      float* coef, float* maximum, const int* row_seq, const int* seq_slot,
                                      const int* seq_row0, const int* seq_len, int seqs, int heads,
                                      cudaStream_t stream) {
    if (seqs <= 0) return 0;
    if (heads <= 0 || !(cap > 0.f)) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)(((long long)seqs * heads * 32 + 127) / 128);
    if (dtype == KIDI_F32)
        return kidi_launch(matrix_memory_gates_kernel<float>, blocks, 128, 0, stream, (const float*)gates, ld, offset_i,
                           offset_f, cap, coef, maximum, row_seq, seq_slot, seq_row0, seq_len, seqs, heads);
    if (dtype == KIDI_BF16)
        return kidi_launch(matrix_memory_gates_kernel<bf16>, blocks, 128, 0, stream, (const bf16*)gates, ld, offset_i,
                           offset_f, cap, coef, maximum, row_seq, seq_slot, seq_row0, seq_len, seqs, heads);
    return KIDI_REFUSED_DTYPE;
}

KIDI_API int kidi_matrix_memory_finish(const float* read, const float* coef, const float* weight, const void* gate,
                                       long long ldg, int dtype, void* out, long long ldo, int rows, int heads, int vdim,
                                       float eps, cudaStream_t stream) {
    const long long items = (long long)rows * heads;
    if (items <= 0) return 0;
    if (vdim <= 0) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)((items * 32 + 127) / 128);
    if (dtype == KIDI_F32)
        return kidi_launch(matrix_memory_finish_kernel<float>, blocks, 128, 0, stream, read, coef, weight,
                           (const float*)gate, ldg, (float*)out, ldo, items, heads, vdim, eps);
    if (dtype == KIDI_BF16)
        return kidi_launch(matrix_memory_finish_kernel<bf16>, blocks, 128, 0, stream, read, coef, weight,
                           (const bf16*)gate, ldg, (bf16*)out, ldo, items, heads, vdim, eps);
    return KIDI_REFUSED_DTYPE;
}
