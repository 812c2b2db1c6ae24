// Attention over a cached latent: what a token leaves in the cache is one row [c | k_rot] per layer, c the
// normalised latent (rank values) from which every head's keys and values are linear maps, k_rot a rotated key part
// (rot_dim values) that all heads share. With the key map folded into the query (q_lat = W_uk^T q, per head) a head's
// score against token u is (q_lat . c_u + q_rot . k_rot_u) * scale and its result is the weighted sum of the c_u,
// to which the value map is applied afterwards: one key/value "head" of width rank + rot_dim whose values are the
// first rank entries of its keys.
//
// Two kernels for any element type: `latent_prepare` (RMS norm of the latent, interleaved rotation of the shared key
// part and of the queries' rotated parts, cache write) and `latent_attention` (causal softmax attention of every row
// over its sequence's cached rows). Norm sums, angles, scores, softmax and the weighted sums are 32-bit. The order
// of a row's additions depends on its position only.
#include "common.cuh"

struct LatentPrepareArgs {
    const void* q;          // [rows, ldq]: per head [dim plain | rot_dim to rotate]
    long long ldq;
    void* folded;           // [rows, ldf]: per head [rank (filled by the caller) | rot_dim rotated, written here]
    long long ldf;
    void* kv;               // [rows, ldkv]: [rank latent | rot_dim shared key part], or null (nothing is cached)
    long long ldkv;
    int write_back;         // the normalised latent and the rotated key part also replace the row of kv
    int skip_queries;       // only the cache entries are made
    const float* kv_norm;   // [rank]
    const float* cos_table; // [positions, rotary_dims / 2]
    const float* sin_table;
    const int* row_seq;     // [rows] (-1: padding row, skipped)
    const int* row_pos;
    const int* seq_slot;
    void* cache;            // storage of this schedule entry [pages, 1, page, rank + rot_dim]
    CacheGeometry geometry;
    int rows, heads, dim, rot_dim, rotary_dims, rank;
    float eps;
};

// One warp per (row, unit): units 0..heads-1 are the query heads, unit `heads` is the row's cache entry.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(LatentPrepareArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.skip_queries ? 0 : a.heads;
    const int units = heads + (a.kv ? 1 : 0);
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * units) return;
    const int row = (int)(item / units), unit = (int)(item - (long long)row * units);
    const int seq = a.row_seq[row];
    if (seq < 0) return;
    const int position = a.row_pos[row];
    const int half = a.rotary_dims / 2;
    const float* cosine = a.cos_table + (long long)position * half;
    const float* sine = a.sin_table + (long long)position * half;
    const T* source;
    T* target;
    T* second = nullptr;    // the row of kv, when it is written back
    if (unit < heads) {
        source = (const T*)a.q + row * a.ldq + (long long)unit * (a.dim + a.rot_dim) + a.dim;
        target = (T*)a.folded + row * a.ldf + (long long)unit * (a.rank + a.rot_dim) + a.rank;
    } else {
        T* latent = (T*)a.kv + row * a.ldkv;
        T* cached = (T*)a.cache + cache_row_offset(a.geometry, a.seq_slot[seq], position, 0);
        float square = 0.f;
        for (int c = lane; c < a.rank; c += 32) {
            const float value = to_float(latent[c]);
            square = fmaf(value, value, square);
        }
        const float inv = 1.0f / sqrtf(warp_sum(square) / (float)a.rank + a.eps);
        for (int c = lane; c < a.rank; c += 32) {
            const T normed = from_float<T>(to_float(latent[c]) * inv * a.kv_norm[c]);
            cached[c] = normed;
            if (a.write_back) latent[c] = normed;
        }
        source = latent + a.rank;
        target = cached + a.rank;
        if (a.write_back) second = latent + a.rank;
    }
    // entries 2i and 2i+1 turn by the angle of pair i; entries from rotary_dims on pass unchanged
    for (int i = lane; i < half; i += 32) {
        const float u = to_float(source[2 * i]), v = to_float(source[2 * i + 1]);
        const float c = cosine[i], s = sine[i];
        const T first = from_float<T>(u * c - v * s), other = from_float<T>(v * c + u * s);
        target[2 * i] = first;
        target[2 * i + 1] = other;
        if (second) { second[2 * i] = first; second[2 * i + 1] = other; }   // the lane's own pair: read above
    }
    for (int c = a.rotary_dims + lane; c < a.rot_dim; c += 32) target[c] = source[c];
}

KIDI_API int kidi_latent_prepare(const LatentPrepareArgs* args, int dtype, cudaStream_t stream) {
    const LatentPrepareArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.skip_queries && !a.kv) return 0;
    if (a.heads <= 0 || a.dim < 0 || a.rot_dim < 0 || a.rank <= 0 || a.rotary_dims < 0 || (a.rotary_dims & 1) ||
        a.rotary_dims > a.rot_dim)
        return KIDI_REFUSED_SIZE;
    const long long items = (long long)a.rows * ((a.skip_queries ? 0 : a.heads) + (a.kv ? 1 : 0));
    if ((items + 3) / 4 > 0x7fffffffLL) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == KIDI_F32) return kidi_launch(latent_prepare_kernel<float>, blocks, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(latent_prepare_kernel<bf16>, blocks, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
struct LatentAttentionArgs {
    const void* folded;     // [rows, ldf]: per head [q_lat (rank) | q_rot (rot_dim)]
    long long ldf;
    const void* cache;      // [pages, 1, page, rank + rot_dim]
    CacheGeometry geometry;
    void* out;              // [rows, ldo]: per head the weighted sum of the latents (rank values)
    long long ldo;
    const int* row_seq;     // [rows] (-1: padding row: output zeros)
    const int* row_pos;
    const int* seq_slot;
    int rows, heads, rank, rot_dim, window;   // window 0: every earlier token is visible
    float scale;
};

// One block of 4 warps per (row, head). Warp w takes tokens first+w, first+w+4, ... in ascending order with an
// online softmax; the four partial results are merged in warp order. CHUNKS * 32 >= rank + rot_dim.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(128) latent_attention_kernel(LatentAttentionArgs a) {
    __shared__ float query[CHUNKS * 32];
    __shared__ float part_acc[4][CHUNKS * 32];
    __shared__ float part_max[4], part_sum[4];
    const int row = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int width = a.rank + a.rot_dim;
    T* out = (T*)a.out + row * a.ldo + (long long)head * a.rank;
    const int seq = a.row_seq[row];
    if (seq < 0) {
        for (int c = threadIdx.x; c < a.rank; c += 128) out[c] = from_float<T>(0.f);
        return;
    }
    const int position = a.row_pos[row];
    const int first = a.window > 0 ? max(0, position - a.window + 1) : 0;
    const int slot = a.seq_slot[seq];
    const T* q = (const T*)a.folded + row * a.ldf + (long long)head * width;
    for (int c = threadIdx.x; c < CHUNKS * 32; c += 128) query[c] = c < width ? to_float(q[c]) : 0.f;
    __syncthreads();

    float best = -INFINITY, denom = 0.f;
    float acc[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) acc[i] = 0.f;
    for (int u = first + warp; u <= position; u += 4) {
        const T* entry = (const T*)a.cache + cache_row_offset(a.geometry, slot, u, 0);
        float kept[CHUNKS];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
            const int c = lane + 32 * i;
            kept[i] = c < width ? to_float(entry[c]) : 0.f;
            dot = fmaf(query[c], kept[i], dot);       // both are zero beyond `width`
        }
        const float score = warp_sum(dot) * a.scale;
        const float next = fmaxf(best, score);
        const float keep = expf(best - next);  // 0 on the first token (best = -inf)
        const float weight = expf(score - next);
        denom = denom * keep + weight;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) acc[i] = acc[i] * keep + weight * kept[i];
        best = next;
    }
    if (lane == 0) { part_max[warp] = best; part_sum[warp] = denom; }
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) part_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float top = part_max[0];
#pragma unroll
    for (int w = 1; w < 4; ++w) top = fmaxf(top, part_max[w]);
    float total = 0.f, factor[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        factor[w] = part_max[w] == -INFINITY ? 0.f : expf(part_max[w] - top);
        total += part_sum[w] * factor[w];
    }
    for (int c = threadIdx.x; c < a.rank; c += 128) {
        float value = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) value += part_acc[w][c] * factor[w];
        out[c] = from_float<T>(value / total);
    }
}

template <typename T>
static int launch_latent_attention(const LatentAttentionArgs& a, cudaStream_t stream) {
    const int width = a.rank + a.rot_dim;
    dim3 grid(a.rows, a.heads);
    if (width <= 128) return kidi_launch(latent_attention_kernel<T, 4>, grid, 128, 0, stream, a);
    if (width <= 256) return kidi_launch(latent_attention_kernel<T, 8>, grid, 128, 0, stream, a);
    if (width <= 384) return kidi_launch(latent_attention_kernel<T, 12>, grid, 128, 0, stream, a);
    if (width <= 640) return kidi_launch(latent_attention_kernel<T, 20>, grid, 128, 0, stream, a);
    return KIDI_REFUSED_SIZE;
}

KIDI_API int kidi_latent_attention(const LatentAttentionArgs* args, int dtype, cudaStream_t stream) {
    const LatentAttentionArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.rank <= 0 || a.rot_dim < 0) return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return launch_latent_attention<float>(a, stream);
    if (dtype == KIDI_BF16) return launch_latent_attention<bf16>(a, stream);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
// The unfolded form for prompts: every head's keys and values are computed from the latents of the step's rows
// and packed, with the queries, into the matrix [rows, 3 * heads * D] (D = dim + rot_dim) that the prompt
// attention kernels of grouped-query attention take: heads of [q_plain | q_rot turned], then heads of
// [k_plain | shared rotated key part], then heads of [value | zeros up to D].
struct LatentPackArgs {
    const void* q;          // [rows, ldq]: per head [dim | rot_dim not yet turned]
    long long ldq;
    const void* latent;     // [rows, ldl]: [rank normalised | rot_dim turned] (as the cache holds them)
    long long ldl;
    const void* unfolded;   // [rows, ldu]: heads*dim plain keys, then heads*vdim values
    long long ldu;
    void* packed;           // [rows, ldp]
    long long ldp;
    const float* cos_table;
    const float* sin_table;
    const int* row_seq;
    const int* row_pos;
    int rows, heads, dim, rot_dim, rotary_dims, rank, vdim;
};

template <typename T>
__global__ void __launch_bounds__(128) latent_pack_kernel(LatentPackArgs a) {
    const int row = blockIdx.x;
    const int D = a.dim + a.rot_dim, half = a.rotary_dims / 2;
    const int position = a.row_seq[row] < 0 ? 0 : a.row_pos[row];
    const float* cosine = a.cos_table + (long long)position * half;
    const float* sine = a.sin_table + (long long)position * half;
    const T* q = (const T*)a.q + row * a.ldq;
    const T* latent = (const T*)a.latent + row * a.ldl;
    const T* unfolded = (const T*)a.unfolded + row * a.ldu;
    T* packed = (T*)a.packed + row * a.ldp;
    const int per_section = a.heads * D;
    for (int index = threadIdx.x; index < 3 * per_section; index += 128) {
        const int section = index / per_section, within = index - section * per_section;
        const int head = within / D, c = within - head * D;
        T value;
        if (section == 0) {
            const T* source = q + head * D;
            if (c < a.dim || c >= a.dim + a.rotary_dims) {
                value = source[c];
            } else {
                const int j = c - a.dim, i = j >> 1;
                const float u = to_float(source[a.dim + 2 * i]), v = to_float(source[a.dim + 2 * i + 1]);
                value = from_float<T>((j & 1) ? v * cosine[i] + u * sine[i] : u * cosine[i] - v * sine[i]);
            }
        } else if (section == 1) {
            value = c < a.dim ? unfolded[head * a.dim + c] : latent[a.rank + c - a.dim];
        } else {
            value = c < a.vdim ? unfolded[a.heads * a.dim + head * a.vdim + c] : from_float<T>(0.f);
        }
        packed[index] = value;
    }
}

// The same in 16-byte pieces (bfloat16; every width a multiple of 8, rows 16-byte aligned): a piece never
// straddles two parts of a head, and a rotated piece holds four whole pairs.
__global__ void __launch_bounds__(256) latent_pack_bf16x8_kernel(LatentPackArgs a) {
    const int row = blockIdx.x;
    const int D = a.dim + a.rot_dim, half = a.rotary_dims / 2;
    const int position = a.row_seq[row] < 0 ? 0 : a.row_pos[row];
    const float* cosine = a.cos_table + (long long)position * half;
    const float* sine = a.sin_table + (long long)position * half;
    const bf16* q = (const bf16*)a.q + row * a.ldq;
    const bf16* latent = (const bf16*)a.latent + row * a.ldl;
    const bf16* unfolded = (const bf16*)a.unfolded + row * a.ldu;
    bf16* packed = (bf16*)a.packed + row * a.ldp;
    const int per_head = D / 8, per_section = a.heads * per_head;
    for (int piece = threadIdx.x; piece < 3 * per_section; piece += 256) {
        const int section = piece / per_section, within = piece - section * per_section;
        const int head = within / per_head, c = (within - head * per_head) * 8;
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (section == 0) {
            value = *reinterpret_cast<const uint4*>(q + head * D + c);
            if (c >= a.dim && c < a.dim + a.rotary_dims) {
                const int i = (c - a.dim) >> 1;
                const float4 cs = *reinterpret_cast<const float4*>(cosine + i), sn = *reinterpret_cast<const float4*>(sine + i);
                const float c4[4] = {cs.x, cs.y, cs.z, cs.w}, s4[4] = {sn.x, sn.y, sn.z, sn.w};
                __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&value);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 uv = __bfloat1622float2(pairs[e]);
                    pairs[e] = __floats2bfloat162_rn(uv.x * c4[e] - uv.y * s4[e], uv.y * c4[e] + uv.x * s4[e]);
                }
            }
        } else if (section == 1) {
            value = c < a.dim ? *reinterpret_cast<const uint4*>(unfolded + head * a.dim + c)
                              : *reinterpret_cast<const uint4*>(latent + a.rank + c - a.dim);
        } else if (c < a.vdim) {
            value = *reinterpret_cast<const uint4*>(unfolded + a.heads * a.dim + head * a.vdim + c);
        }
        *reinterpret_cast<uint4*>(packed + (long long)piece * 8) = value;
    }
}

KIDI_API int kidi_latent_pack(const LatentPackArgs* args, int dtype, cudaStream_t stream) {
    const LatentPackArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads <= 0 || a.vdim > a.dim + a.rot_dim || a.rotary_dims > a.rot_dim || (a.rotary_dims & 1)) return KIDI_REFUSED_SIZE;
    const bool pieces = dtype == KIDI_BF16 && !((a.dim | a.rot_dim | a.vdim | a.rank | a.rotary_dims) & 7) &&
                        !((a.ldq | a.ldl | a.ldu | a.ldp) & 7) && !(((uintptr_t)a.q | (uintptr_t)a.latent |
                        (uintptr_t)a.unfolded | (uintptr_t)a.packed | (uintptr_t)a.cos_table | (uintptr_t)a.sin_table) & 15);
    if (pieces) return kidi_launch(latent_pack_bf16x8_kernel, a.rows, 256, 0, stream, a);
    if (dtype == KIDI_F32) return kidi_launch(latent_pack_kernel<float>, a.rows, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(latent_pack_kernel<bf16>, a.rows, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// Rows of the step as the cache holds them: out[r] = the cached entry of row r's sequence at row r's position
// (for a layer that reads another layer's cached rows). Padding rows get zeros.
template <typename T>
__global__ void __launch_bounds__(128)
latent_gather_kernel(const T* __restrict__ cache, CacheGeometry geometry, T* __restrict__ out, long long ldo,
                     const int* __restrict__ row_seq, const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                     int width) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    T* target = out + row * ldo;
    if (seq < 0) {
        for (int c = threadIdx.x; c < width; c += 128) target[c] = from_float<T>(0.f);
        return;
    }
    const T* entry = cache + cache_row_offset(geometry, seq_slot[seq], row_pos[row], 0);
    for (int c = threadIdx.x; c < width; c += 128) target[c] = entry[c];
}

KIDI_API int kidi_latent_gather(const void* cache, const CacheGeometry* geometry, void* out, long long ldo,
                                const int* row_seq, const int* row_pos, const int* seq_slot, int rows, int width,
                                int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == KIDI_F32)
        return kidi_launch(latent_gather_kernel<float>, rows, 128, 0, stream, (const float*)cache, *geometry,
                           (float*)out, ldo, row_seq, row_pos, seq_slot, width);
    if (dtype == KIDI_BF16)
        return kidi_launch(latent_gather_kernel<bf16>, rows, 128, 0, stream, (const bf16*)cache, *geometry, (bf16*)out,
                           ldo, row_seq, row_pos, seq_slot, width);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
// The folded form on the tensor cores (bfloat16; rank and rot_dim multiples of 16, rank <= 512, pages of 64
// tokens, every page kept; a window is a mask and the first page of the walk). A block of eight warps takes one row of the step, a tile of up to 16 of its heads and a share
// of its sequence's pages. A page [64 tokens, W = rank + rot_dim] is copied to shared memory once (cp.async) and
// serves as the keys of S = Q K^T (all W columns) and, its first `rank` columns, as the values of O += P C: the
// cached rows are read once for all heads of the tile. Warp w of eight computes the scores of the page's tokens
// 8w..8w+7 for the 16 heads (`mma.sync` m16n8k16, fragments by `ldmatrix`), the warps exchange row maxima and sums through
// shared memory (online softmax in 32-bit), P goes to shared memory in bfloat16, and warp w accumulates the output
// columns of its n-tiles (tile i belongs to warp i mod 8) with the page as a transposed B operand
// (`ldmatrix.trans`). Every block leaves (O, max, sum) of its share in a workspace; `latent_combine` merges the
// shares of a (row, head) in their order.
struct LatentDecodeArgs {
    const void* folded;     // [rows, ldf]: per head [q_lat (rank) | q_rot (rot_dim)], bfloat16
    long long ldf;
    const void* cache;      // [pages, 64, W] bfloat16
    const int* table;       // [slots, pages_per_seq]
    int pages_per_seq;
    const int* row_seq;
    const int* row_pos;
    const int* seq_slot;
    float* part_o;          // [rows, splits, heads, rank]
    float* part_stat;       // [rows, splits, heads, 2]: max, sum
    void* out;              // [rows, ldo] bfloat16 (combine)
    long long ldo;
    int rows, heads, rank, rot_dim, splits;
    float scale;
    int splits_are_long;    // > 0: a share holds several pages: worth a second page buffer even at one block an
                            // SM; < 0: one page buffer whatever the sizes
    int window;             // > 0: a row at position p sees the tokens p - window + 1 .. p only
};

namespace {
__device__ __forceinline__ unsigned shared_address(const void* pointer) {
    return (unsigned)__cvta_generic_to_shared(pointer);
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void copy_async_16(unsigned destination, const void* source) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source));
}

constexpr int PAGE = 64;

constexpr int WARPS = 8;

template <int TILES, int BUFFERS>   // output n-tiles (8 columns) a warp owns at most: rank <= 64 * TILES; page buffers
__global__ void __launch_bounds__(32 * WARPS) latent_decode_kernel(LatentDecodeArgs a) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int row = blockIdx.x, head0 = blockIdx.y * 16, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int W = a.rank + a.rot_dim, stride = W + 8;      // padded rows: ldmatrix without bank conflicts
    bf16* Qs = reinterpret_cast<bf16*>(raw);                // [16][stride]
    bf16* pages_at = Qs + 16 * stride;                      // [BUFFERS][64][stride]
    bf16* Ps = pages_at + BUFFERS * PAGE * stride;          // [16][PAGE + 8]
    float* wmax = reinterpret_cast<float*>(Ps + 16 * (PAGE + 8));   // [WARPS][16]
    float* wsum = wmax + WARPS * 16;                        // [WARPS][16]
    const int heads_here = min(16, a.heads - head0);
    float* part_o = a.part_o + (((long long)row * a.splits + split) * a.heads + head0) * a.rank;
    float* part_stat = a.part_stat + (((long long)row * a.splits + split) * a.heads + head0) * 2;
    const int seq = a.row_seq[row];
    int first_page = 0, last_page = 0, position = -1, slot = 0;
    if (seq >= 0) {
        position = a.row_pos[row];
        slot = a.seq_slot[seq];
        const int pages = (position >> 6) + 1;
        const int low_page = a.window > 0 ? max(0, position - a.window + 1) >> 6 : 0;   // the first page with a visible token
        const int per = (pages - low_page + a.splits - 1) / a.splits;
        first_page = low_page + split * per;
        last_page = min(pages, first_page + per);
    }
    if (first_page >= last_page) {                          // nothing to do: an empty share
        if (threadIdx.x < heads_here) {
            part_stat[threadIdx.x * 2] = -INFINITY;
            part_stat[threadIdx.x * 2 + 1] = 0.f;
        }
        return;
    }
    // the tile's queries (zero rows beyond the heads) travel with the first page
    const bf16* q = (const bf16*)a.folded + row * a.ldf + (long long)head0 * W;
    for (int h = warp; h < 16; h += WARPS)
        for (int c = lane * 8; c < W; c += 256) {
            if (h < heads_here) copy_async_16(shared_address(Qs + h * stride + c), q + (long long)h * W + c);
            else *reinterpret_cast<uint4*>(Qs + h * stride + c) = make_uint4(0u, 0u, 0u, 0u);
        }
    float o[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float best[2] = {-INFINITY, -INFINITY}, denom[2] = {0.f, 0.f};   // of rows g and g + 8
    const int n_tiles = a.rank / 8;
    // a page of the cache into one of the buffers, 16 bytes a copy
    auto copy_page = [&](int page_index, bf16* target) {
        const int page = a.table[(long long)slot * a.pages_per_seq + page_index];
        const bf16* source = (const bf16*)a.cache + (long long)page * PAGE * W;
        for (int r = warp; r < PAGE; r += WARPS)
            for (int c = lane * 8; c < W; c += 256)
                copy_async_16(shared_address(target + r * stride + c), source + (long long)r * W + c);
        asm volatile("cp.async.commit_group;");
    };
    copy_page(first_page, pages_at);
    for (int page_index = first_page; page_index < last_page; ++page_index) {
        const bf16* Ks = pages_at + ((page_index - first_page) % BUFFERS) * PAGE * stride;
        asm volatile("cp.async.wait_group 0;");
        __syncthreads();                                    // this page has landed; the last page's products are done
        if (BUFFERS > 1) {
            if (page_index + 1 < last_page)                 // the next page travels while this one is computed
                copy_page(page_index + 1, pages_at + ((page_index + 1 - first_page) % BUFFERS) * PAGE * stride);
        }
        // scores of tokens 8 warp .. 8 warp + 7 against the 16 heads: two k-steps a round, each with an
        // accumulator of its own, so that neither the loads nor the products wait for one another
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s_other[4] = {0.f, 0.f, 0.f, 0.f};
        const unsigned q_at = shared_address(Qs + (lane & 15) * stride + (lane >> 4) * 8);
        const unsigned k_at = shared_address(Ks + (8 * warp + (lane & 7)) * stride + (lane >> 3) * 8);
        int k0 = 0;
#pragma unroll 2
        for (; k0 + 32 <= W; k0 += 32) {
            unsigned qa[4], qb[4], kb[4];
            ldmatrix_x4(kb, k_at + k0 * 2);                 // (k0..7, 8..15, 16..23, 24..31) of the warp's 8 tokens
            ldmatrix_x4(qa, q_at + k0 * 2);
            ldmatrix_x4(qb, q_at + (k0 + 16) * 2);
            mma_bf16(s, qa, kb[0], kb[1]);
            mma_bf16(s_other, qb, kb[2], kb[3]);
        }
        if (k0 < W) {                                       // a last k-step of 16: the upper two matrices are re-read
            unsigned qa[4], kb[4];
            ldmatrix_x4(kb, shared_address(Ks + (8 * warp + (lane & 7)) * stride + k0 + ((lane >> 3) & 1) * 8));
            ldmatrix_x4(qa, q_at + k0 * 2);
            mma_bf16(s, qa, kb[0], kb[1]);
        }
        const int token0 = page_index * PAGE + 8 * warp + 2 * t;
        float top[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int token = token0 + (e & 1);
            const bool seen = token <= position && (a.window <= 0 || token > position - a.window);
            s[e] = seen ? (s[e] + s_other[e]) * a.scale : -INFINITY;
            top[e >> 1] = fmaxf(top[e >> 1], s[e]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
            top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
        }
        if (t == 0) { wmax[warp * 16 + g] = top[0]; wmax[warp * 16 + g + 8] = top[1]; }
        __syncthreads();
        float next[2], keep[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int h = g + 8 * r;
            float tile = wmax[h];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) tile = fmaxf(tile, wmax[w * 16 + h]);
            next[r] = fmaxf(best[r], tile);                 // finite: every page of the walk holds a token that the row sees
            keep[r] = expf(best[r] - next[r]);              // 0 on the first page
        }
        {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = expf(s[e] - next[e >> 1]);
                sum[e >> 1] += p[e];
            }
            const int column = 8 * warp + 2 * t;
            *reinterpret_cast<__nv_bfloat162*>(Ps + g * (PAGE + 8) + column) = __floats2bfloat162_rn(p[0], p[1]);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * (PAGE + 8) + column) = __floats2bfloat162_rn(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        }
        if (t == 0) { wsum[warp * 16 + g] = sum[0]; wsum[warp * 16 + g + 8] = sum[1]; }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int h = g + 8 * r;
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) total += wsum[w * 16 + h];
            denom[r] = denom[r] * keep[r] + total;
            best[r] = next[r];
        }
        // O = O * keep + P C over this warp's n-tiles (tile n belongs to warp n mod WARPS)
        unsigned pa[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            ldmatrix_x4(pa[k], shared_address(Ps + (lane & 15) * (PAGE + 8) + 16 * k + (lane >> 4) * 8));
#pragma unroll
        for (int i = 0; i < TILES; i += 2) {                // two n-tiles a ldmatrix
            const int n_first = warp + WARPS * i, n_second = warp + WARPS * (i + 1);
            if (n_first < n_tiles) {
                o[i][0] *= keep[0]; o[i][1] *= keep[0]; o[i][2] *= keep[1]; o[i][3] *= keep[1];
                o[i + 1][0] *= keep[0]; o[i + 1][1] *= keep[0]; o[i + 1][2] *= keep[1]; o[i + 1][3] *= keep[1];
                const bool both = n_second < n_tiles;
                const int mi = lane >> 3;
                const int column = ((mi >> 1) && both ? n_second : n_first) * 8;
                unsigned cb[4][4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    ldmatrix_x4_trans(cb[k], shared_address(Ks + (16 * k + (mi & 1) * 8 + (lane & 7)) * stride + column));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_bf16(o[i], pa[k], cb[k][0], cb[k][1]);
                    if (both) mma_bf16(o[i + 1], pa[k], cb[k][2], cb[k][3]);
                }
            }
        }
        if (BUFFERS == 1 && page_index + 1 < last_page) {
            __syncthreads();                                // one buffer: the next page may only be copied now
            copy_page(page_index + 1, pages_at);
        }
    }
    // this share's result
#pragma unroll
    for (int i = 0; i < TILES; ++i) {
        const int n = warp + WARPS * i;
        if (n < n_tiles) {
            const int column = n * 8 + 2 * t;
            if (g < heads_here)
                *reinterpret_cast<float2*>(part_o + (long long)g * a.rank + column) = make_float2(o[i][0], o[i][1]);
            if (g + 8 < heads_here)
                *reinterpret_cast<float2*>(part_o + (long long)(g + 8) * a.rank + column) = make_float2(o[i][2], o[i][3]);
        }
    }
    if (warp == 0 && t == 0) {
        if (g < heads_here) { part_stat[g * 2] = best[0]; part_stat[g * 2 + 1] = denom[0]; }
        if (g + 8 < heads_here) { part_stat[(g + 8) * 2] = best[1]; part_stat[(g + 8) * 2 + 1] = denom[1]; }
    }
}

// out[row, head, :] = sum_s w_s O_s / sum_s w_s l_s with w_s = exp(max_s - max), over the shares in their order.
__global__ void __launch_bounds__(128) latent_combine_kernel(LatentDecodeArgs a) {
    const int row = blockIdx.x, head = blockIdx.y;
    bf16* out = (bf16*)a.out + row * a.ldo + (long long)head * a.rank;
    const float* stat = a.part_stat + ((long long)row * a.splits * a.heads + head) * 2;
    const float* part = a.part_o + ((long long)row * a.splits * a.heads + head) * a.rank;
    const long long step = (long long)a.heads;
    float top = -INFINITY;
    for (int s = 0; s < a.splits; ++s) top = fmaxf(top, stat[s * step * 2]);
    if (a.row_seq[row] < 0 || top == -INFINITY) {
        for (int c = threadIdx.x; c < a.rank; c += 128) out[c] = from_float<bf16>(0.f);
        return;
    }
    float total = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const float m = stat[s * step * 2];
        if (m != -INFINITY) total += stat[s * step * 2 + 1] * expf(m - top);
    }
    for (int c = threadIdx.x; c < a.rank; c += 128) {
        float value = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float m = stat[s * step * 2];
            if (m != -INFINITY) value += part[s * step * a.rank + c] * expf(m - top);
        }
        out[c] = from_float<bf16>(value / total);
    }
}

template <int TILES, int BUFFERS>
int launch_decode_form(const LatentDecodeArgs& a, size_t shared, cudaStream_t stream) {
    auto kernel = latent_decode_kernel<TILES, BUFFERS>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    dim3 grid(a.rows, (a.heads + 15) / 16, a.splits);
    const int status = kidi_launch(kernel, grid, 32 * WARPS, shared, stream, a);
    if (status) return status;
    return kidi_launch(latent_combine_kernel, dim3(a.rows, a.heads), 128, 0, stream, a);
}

template <int TILES>
int launch_decode(const LatentDecodeArgs& a, cudaStream_t stream) {
    const int W = a.rank + a.rot_dim;
    const size_t rest = (size_t)16 * (W + 8) * 2 + 16 * (PAGE + 8) * 2 + 2 * WARPS * 16 * sizeof(float);
    const size_t page = (size_t)PAGE * (W + 8) * 2;
    // two page buffers (the next page is copied while this one is computed) where they leave room for two blocks
    // an SM or the share has several pages anyway; else one
    if (a.splits_are_long >= 0 && rest + 2 * page <= 110 * 1024) return launch_decode_form<TILES, 2>(a, rest + 2 * page, stream);
    if (rest + 2 * page <= 220 * 1024 && a.splits_are_long > 0) return launch_decode_form<TILES, 2>(a, rest + 2 * page, stream);
    return launch_decode_form<TILES, 1>(a, rest + page, stream);
}
}  // namespace

// How many floats of workspace a launch needs (part_o, then part_stat).
KIDI_API long long kidi_latent_decode_workspace(int rows, int heads, int rank, int splits) {
    return (long long)rows * splits * heads * (rank + 2);
}

KIDI_API int kidi_latent_decode(const LatentDecodeArgs* args, cudaStream_t stream) {
    const LatentDecodeArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads <= 0 || (a.heads + 15) / 16 > 65535 || a.splits <= 0 || a.splits > 65535 || a.rank <= 0 || (a.rank & 15) ||
        (a.rot_dim & 15) || a.rank > 512 || a.rot_dim < 0 || a.rank + a.rot_dim > 1024 || (a.ldf & 7) ||
        ((uintptr_t)a.folded & 15) || ((uintptr_t)a.cache & 15))
        return KIDI_REFUSED_SIZE;
    if (a.rank <= 128) return launch_decode<2>(a, stream);
    if (a.rank <= 256) return launch_decode<4>(a, stream);
    return launch_decode<8>(a, stream);
}
