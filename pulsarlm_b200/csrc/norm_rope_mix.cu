// What lies between an attention layer's projections and its attention, for layers whose
// queries and keys are normed, whose key and value sizes may differ, and whose values may be
// mixed with those of an earlier layer. One launch per layer and step, per token:
//
//   q, k: an RMS norm in one of four ways (none; per head over its `dim` columns with one
//         weight row shared by the heads; over the whole projection, all heads at once, with
//         a weight per column; per head without weights AFTER the rotation), and a
//         rotate-half rotation of the first `rotary` columns of every head in between
//         (angle in fp64 from an fp64 table, reduced, sincos in fp32, as rope_kv.cu);
//   v:    v <- (1 - lambda) v + lambda v_first, where v_first holds another layer's values
//         of the same token (nullptr: no mixing);
//   then q goes to q_out [T, heads, row] and k and v into the token's place in the paged
//   cache, both as rows of the common size `row` >= max(dim, vdim) with zeros past their own
//   columns, so that the paged attention kernels (one row size for q, k and v) run them as
//   they are: a product with a zero adds nothing.
//
// Statistics, norm products, rotation and the mix are fp32, one rounding on each store. Two
// kernels: one that keeps a head's row in the registers of a group of lanes, eight columns a lane
// (sizes in multiples of eight on 16-byte addresses: the usual case), and one that walks a head
// column by column for every other shape. Which of them runs, and the order in which either adds
// up a token's sums, depends on the sizes alone, never on the step.
#include "rope_helpers.cuh"

namespace {

enum NormMode : int { kNone = 0, kPerHead = 1, kWhole = 2, kUnitAfter = 3 };
constexpr int kThreads = 128;

template <typename scalar_t>
__global__ void __launch_bounds__(kThreads)
norm_rope_mix_write_kernel(const scalar_t* __restrict__ q, const scalar_t* __restrict__ k,
                           const scalar_t* __restrict__ v, int64_t row_stride,
                           const scalar_t* __restrict__ v_first, int64_t v_first_stride, float lambda,
                           scalar_t* __restrict__ q_out, const int32_t* __restrict__ pos,
                           const int32_t* __restrict__ entry, const int32_t* __restrict__ table, int table_width,
                           scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool, int64_t page_stride,
                           int64_t head_stride, int page_size, int n_pages, const double* __restrict__ inv_freq,
                           int rotary, int n_heads, int n_kv, int dim, int vdim, int row, int heads_per_block,
                           int mode, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                           float eps, int32_t* status) {
    extern __shared__ float shared[];  // [rotary] cos | sin, [32] scratch, [warps][dim] a head's columns
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = shared;
    float* sn = shared + half;
    float* scratch = shared + rotary;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kThreads / 32;
    float* buf = scratch + 32 + warp * dim;
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += kThreads) {
            rope_sincos(p, inv_freq[j], cs[j], sn[j]);
        }
    }
    const int n_slots = n_heads + 2 * n_kv;
    const int slot0 = blockIdx.y * heads_per_block;
    const int slot1 = min(slot0 + heads_per_block, n_slots);
    int page = -1;
    if (slot1 > n_heads) {
        page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && status != nullptr) {
                atomicOr(status, 2);
            }
            page = -1;
        }
    }
    float whole_q = 1.0f, whole_k = 1.0f;
    if (mode == kWhole) {
        // (uniform over the block: both conditions depend on the block's slots only)
        if (slot0 < n_heads) {
            float sum = 0.0f;
            for (int i = threadIdx.x; i < n_heads * dim; i += kThreads) {
                const float x = pl_load(q + t * row_stride + i);
                sum = fmaf(x, x, sum);
            }
            whole_q = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(n_heads * dim) + eps);
        }
        if (slot1 > n_heads && slot0 < n_heads + n_kv) {
            float sum = 0.0f;
            for (int i = threadIdx.x; i < n_kv * dim; i += kThreads) {
                const float x = pl_load(k + t * row_stride + i);
                sum = fmaf(x, x, sum);
            }
            whole_k = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(n_kv * dim) + eps);
        }
    }
    __syncthreads();

    for (int slot = slot0 + warp; slot < slot1; slot += warps) {
        if (slot >= n_heads + n_kv) {
            // a value head: mixed, stored, zeros up to the row's end
            if (page < 0) {
                continue;
            }
            const int h = slot - n_heads - n_kv;
            const scalar_t* y = v + t * row_stride + static_cast<int64_t>(h) * vdim;
            const scalar_t* f = v_first != nullptr ? v_first + t * v_first_stride + static_cast<int64_t>(h) * vdim : nullptr;
            scalar_t* to = v_pool + page * page_stride + h * head_stride + static_cast<int64_t>(p % page_size) * row;
            for (int d = lane; d < row; d += 32) {
                float value = 0.0f;
                if (d < vdim) {
                    value = pl_load(y + d);
                    if (f != nullptr) {
                        value = __fmaf_rn(lambda, pl_load(f + d), __fmul_rn(1.0f - lambda, value));
                    }
                }
                pl_store(to + d, value);
            }
            continue;
        }
        const bool is_q = slot < n_heads;
        const int h = is_q ? slot : slot - n_heads;
        if (!is_q && page < 0) {
            continue;
        }
        const scalar_t* x = (is_q ? q : k) + t * row_stride + static_cast<int64_t>(h) * dim;
        const float* weight = is_q ? q_weight : k_weight;
        if (weight != nullptr && mode == kWhole) {
            weight += static_cast<int64_t>(h) * dim;
        }
        __syncwarp();
        float sum = 0.0f;
        for (int d = lane; d < dim; d += 32) {
            const float value = pl_load(x + d);
            buf[d] = value;
            sum = fmaf(value, value, sum);
        }
        float r = 1.0f;
        if (mode == kPerHead) {
            r = rsqrtf(pl_warp_sum(sum) / static_cast<float>(dim) + eps);
        } else if (mode == kWhole) {
            r = is_q ? whole_q : whole_k;
        }
        if (mode == kPerHead || mode == kWhole) {
            for (int d = lane; d < dim; d += 32) {
                const float scaled = buf[d] * r;
                buf[d] = weight != nullptr ? scaled * weight[d] : scaled;
            }
        }
        __syncwarp();
        if (inv_freq != nullptr) {
            for (int j = lane; j < half; j += 32) {
                const float lo = buf[j], hi = buf[j + half];
                buf[j] = rope_lo(lo, hi, cs[j], sn[j]);
                buf[j + half] = rope_hi(lo, hi, cs[j], sn[j]);
            }
            __syncwarp();
        }
        float after = 1.0f;
        if (mode == kUnitAfter) {
            float sum2 = 0.0f;
            for (int d = lane; d < dim; d += 32) {
                sum2 = fmaf(buf[d], buf[d], sum2);
            }
            after = rsqrtf(pl_warp_sum(sum2) / static_cast<float>(dim) + eps);
        }
        scalar_t* to = is_q ? q_out + (static_cast<int64_t>(t) * n_heads + h) * row
                            : k_pool + page * page_stride + h * head_stride + static_cast<int64_t>(p % page_size) * row;
        for (int d = lane; d < row; d += 32) {
            pl_store(to + d, d < dim ? buf[d] * after : 0.0f);
        }
    }
}

// Sixteen bytes of a row as floats.
template <typename scalar_t>
struct Piece;
template <>
struct Piece<float> {
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ static __forceinline__ void store(float* p, const float* in) {
        *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    }
};
template <>
struct Piece<__nv_bfloat16> {
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(words[i] << 16);
            out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ void store(__nv_bfloat16* p, const float* in) {
        uint4 raw;
        uint32_t* words = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
            words[i] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// The same with sixteen bytes (bfloat16) or thirty-two (float32) a lane: eight columns. A head's row of the
// common size is shared out over a group of `lanes` neighbouring lanes (a power of two, at least row / 8), so a
// warp works on 32 / lanes heads at once, everything in registers: sums of squares inside the group by
// shuffles, the rotation's partner columns (rotary / 2 columns away: a whole number of lanes) by a shuffle a
// column. Every lane runs the same shuffles whatever its head is (a query, a key or a value head). Takes key,
// value and row sizes and half the rotary width that are multiples of 8. The sums' order depends on the sizes
// alone: a lane's eight columns in turn, then the group's lanes as a tree; a whole projection by the block's
// 128 threads, eight columns a thread and turn, then the block's tree.
template <typename scalar_t>
__global__ void __launch_bounds__(kThreads)
norm_rope_mix_write_pieces_kernel(const scalar_t* __restrict__ q, const scalar_t* __restrict__ k,
                                  const scalar_t* __restrict__ v, int64_t row_stride,
                                  const scalar_t* __restrict__ v_first, int64_t v_first_stride, float lambda,
                                  scalar_t* __restrict__ q_out, const int32_t* __restrict__ pos,
                                  const int32_t* __restrict__ entry, const int32_t* __restrict__ table,
                                  int table_width, scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool,
                                  int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                  const double* __restrict__ inv_freq, int rotary, int n_heads, int n_kv, int dim,
                                  int vdim, int row, int heads_per_block, int lanes, int mode,
                                  const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                  int32_t* status) {
    extern __shared__ float shared[];  // [rotary] cos | sin, [32] scratch
    constexpr int kCols = 8;
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = shared;
    float* sn = shared + half;
    float* scratch = shared + rotary;
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += kThreads) {
            rope_sincos(p, inv_freq[j], cs[j], sn[j]);
        }
    }
    const int n_slots = n_heads + 2 * n_kv;
    const int slot0 = blockIdx.y * heads_per_block;
    const int slot1 = min(slot0 + heads_per_block, n_slots);
    int page = -1;
    if (slot1 > n_heads) {
        page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && status != nullptr) {
                atomicOr(status, 2);
            }
            page = -1;
        }
    }
    auto load8 = [](const scalar_t* from, float* x) {
        if constexpr (sizeof(scalar_t) == 2) {
            Piece<scalar_t>::load(from, x);
        } else {
            Piece<scalar_t>::load(from, x);
            Piece<scalar_t>::load(from + 4, x + 4);
        }
    };
    auto store8 = [](scalar_t* to, const float* x) {
        if constexpr (sizeof(scalar_t) == 2) {
            Piece<scalar_t>::store(to, x);
        } else {
            Piece<scalar_t>::store(to, x);
            Piece<scalar_t>::store(to + 4, x + 4);
        }
    };
    float whole_q = 1.0f, whole_k = 1.0f;
    if (mode == kWhole) {
        // (uniform over the block: both conditions depend on the block's slots only)
        if (slot0 < n_heads) {
            float sum = 0.0f;
            for (int i = threadIdx.x * kCols; i < n_heads * dim; i += kThreads * kCols) {
                float x[kCols];
                load8(q + t * row_stride + i, x);
#pragma unroll
                for (int u = 0; u < kCols; ++u) {
                    sum = fmaf(x[u], x[u], sum);
                }
            }
            whole_q = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(n_heads * dim) + eps);
        }
        if (slot1 > n_heads && slot0 < n_heads + n_kv) {
            float sum = 0.0f;
            for (int i = threadIdx.x * kCols; i < n_kv * dim; i += kThreads * kCols) {
                float x[kCols];
                load8(k + t * row_stride + i, x);
#pragma unroll
                for (int u = 0; u < kCols; ++u) {
                    sum = fmaf(x[u], x[u], sum);
                }
            }
            whole_k = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(n_kv * dim) + eps);
        }
    }
    __syncthreads();

    const int groups = kThreads / lanes;
    const int group = threadIdx.x / lanes, li = threadIdx.x % lanes, lane = threadIdx.x & 31;
    const int e0 = li * kCols;
    const int shift = half / kCols;  // lanes between a column and its partner in the rotation
    for (int first = slot0; first < slot1; first += groups) {  // (every thread of the block makes every turn)
        const int slot = first + group;
        const bool valid = slot < slot1;
        const bool is_q = slot < n_heads, is_v = slot >= n_heads + n_kv;
        const int h = is_q ? slot : (is_v ? slot - n_heads - n_kv : slot - n_heads);
        const int own = is_v ? vdim : dim;
        const bool mine = valid && e0 < own && (is_q || page >= 0);
        float x[kCols];
#pragma unroll
        for (int u = 0; u < kCols; ++u) {
            x[u] = 0.0f;
        }
        if (mine) {
            load8((is_q ? q : (is_v ? v : k)) + t * row_stride + static_cast<int64_t>(h) * own + e0, x);
            if (is_v && v_first != nullptr) {
                float f[kCols];
                load8(v_first + t * v_first_stride + static_cast<int64_t>(h) * vdim + e0, f);
#pragma unroll
                for (int u = 0; u < kCols; ++u) {
                    x[u] = __fmaf_rn(lambda, f[u], __fmul_rn(1.0f - lambda, x[u]));
                }
            }
        }
        const bool normed = mine && !is_v;
        if (mode == kPerHead) {
            float sum = 0.0f;
#pragma unroll
            for (int u = 0; u < kCols; ++u) {
                sum = fmaf(x[u], x[u], sum);
            }
            for (int offset = lanes / 2; offset > 0; offset >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, offset);
            }
            if (normed) {
                const float r = rsqrtf(sum / static_cast<float>(dim) + eps);
                const float* weight = is_q ? q_weight : k_weight;
#pragma unroll
                for (int u = 0; u < kCols; ++u) {
                    const float scaled = x[u] * r;
                    x[u] = weight != nullptr ? scaled * weight[e0 + u] : scaled;
                }
            }
        } else if (mode == kWhole && normed) {
            const float r = is_q ? whole_q : whole_k;
            const float* weight = is_q ? q_weight : k_weight;
#pragma unroll
            for (int u = 0; u < kCols; ++u) {
                const float scaled = x[u] * r;
                x[u] = weight != nullptr ? scaled * weight[static_cast<int64_t>(h) * dim + e0 + u] : scaled;
            }
        }
        if (inv_freq != nullptr) {
            const bool low = e0 < half, turns = normed && e0 < rotary;
            const int partner = turns ? (low ? lane + shift : lane - shift) : lane;
#pragma unroll
            for (int u = 0; u < kCols; ++u) {
                const float other = __shfl_sync(0xffffffffu, x[u], partner);
                if (turns) {
                    const int j = (low ? e0 : e0 - half) + u;
                    x[u] = low ? rope_lo(x[u], other, cs[j], sn[j]) : rope_hi(other, x[u], cs[j], sn[j]);
                }
            }
        }
        if (mode == kUnitAfter) {
            float sum = 0.0f;
#pragma unroll
            for (int u = 0; u < kCols; ++u) {
                sum = fmaf(x[u], x[u], sum);
            }
            for (int offset = lanes / 2; offset > 0; offset >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, offset);
            }
            if (normed) {
                const float after = rsqrtf(sum / static_cast<float>(dim) + eps);
#pragma unroll
                for (int u = 0; u < kCols; ++u) {
                    x[u] *= after;
                }
            }
        }
        if (valid && e0 < row && (is_q || page >= 0)) {  // (columns past the head's own are zeros)
            scalar_t* to = is_q ? q_out + (static_cast<int64_t>(t) * n_heads + h) * row
                                : (is_v ? v_pool : k_pool) + page * page_stride + h * head_stride +
                                      static_cast<int64_t>(p % page_size) * row;
            store8(to + e0, x);
        }
    }
}

}  // namespace

// q [T, n_heads, dim], k [T, n_kv, dim], v [T, n_kv, vdim] with `row_stride` elements between
// tokens (slices of one projection's output); v_first [T, n_kv, vdim] with its own stride, or
// nullptr; q_out [T, n_heads, row] contiguous. Pools: element (page, head, place, d) at page *
// page_stride + head * head_stride + place * row + d. mode: 0 no norm, 1 per head before the
// rotation (q_weight, k_weight fp32 [dim] or nullptr), 2 over the whole projection before the
// rotation (q_weight fp32 [n_heads * dim], k_weight fp32 [n_kv * dim], or nullptr), 3 per head
// without weights after the rotation. inv_freq == nullptr: no rotation.
PL_API int pl_norm_rope_mix_write(const void* q, const void* k, const void* v, int64_t row_stride,
                                  const void* v_first, int64_t v_first_stride, float lambda, void* q_out,
                                  const int32_t* pos, const int32_t* entry, const int32_t* table, int table_width,
                                  void* k_pool, void* v_pool, int64_t page_stride, int64_t head_stride,
                                  int page_size, int n_pages, const double* inv_freq, int rotary, int n_tokens,
                                  int n_heads, int n_kv, int dim, int vdim, int row, int mode,
                                  const float* q_weight, const float* k_weight, float eps, int dtype,
                                  int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv > 0 && dim > 0 && vdim > 0 && page_size > 0,
               "norm_rope_mix_write: bad sizes tokens=%d heads=%d kv_heads=%d dim=%d vdim=%d page=%d", n_tokens,
               n_heads, n_kv, dim, vdim, page_size);
    PL_REQUIRE(row >= dim && row >= vdim, "norm_rope_mix_write: a row of %d does not hold keys of %d and values of %d",
               row, dim, vdim);
    PL_REQUIRE(rotary >= 0 && rotary <= dim && rotary % 2 == 0,
               "norm_rope_mix_write: rotary width %d must be even and at most the key size %d", rotary, dim);
    PL_REQUIRE(mode >= kNone && mode <= kUnitAfter, "norm_rope_mix_write: unknown norm mode %d", mode);
    if (n_tokens == 0) {
        return 0;
    }
    const int n_slots = n_heads + 2 * n_kv;
    // Sizes in whole pieces of eight columns, on 16-byte addresses: the kernel that keeps a head in registers.
    const size_t elem = dtype == PL_F32 ? 4 : 2;
    const auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const int64_t step = static_cast<int64_t>(16 / elem);  // elements between addresses 16 bytes apart
    const bool pieces = dim % 8 == 0 && vdim % 8 == 0 && row % 8 == 0 && row <= 256 && (rotary / 2) % 8 == 0 &&
        aligned(q) && aligned(k) && aligned(v) && aligned(q_out) && aligned(k_pool) && aligned(v_pool) &&
        row_stride % step == 0 && page_stride % step == 0 && head_stride % step == 0 &&
        (v_first == nullptr || (aligned(v_first) && v_first_stride % step == 0));
    if (pieces) {
        int lanes = 1;
        while (lanes * 8 < row) {
            lanes *= 2;
        }
        const int groups = kThreads / lanes;
        // few tokens: a block's groups take one head each (many small blocks); long steps: a block per token
        const int heads_per_block = n_tokens >= 256 ? n_slots : groups;
        const size_t smem = (static_cast<size_t>(rotary) + 32) * sizeof(float);
        const dim3 grid(n_tokens, (n_slots + heads_per_block - 1) / heads_per_block);
        PL_REQUIRE(grid.y <= 65535, "norm_rope_mix_write: too many heads (%d)", n_slots);
        PL_DISPATCH_DTYPE(dtype, "norm_rope_mix_write", {
            pl_launch_overlapped(norm_rope_mix_write_pieces_kernel<scalar_t>, grid, dim3(kThreads), smem, stream,
                                 static_cast<const scalar_t*>(q), static_cast<const scalar_t*>(k),
                                 static_cast<const scalar_t*>(v), row_stride, static_cast<const scalar_t*>(v_first),
                                 v_first_stride, lambda, static_cast<scalar_t*>(q_out), pos, entry, table, table_width,
                                 static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool), page_stride,
                                 head_stride, page_size, n_pages, inv_freq, rotary, n_heads, n_kv, dim, vdim, row,
                                 heads_per_block, lanes, mode, q_weight, k_weight, eps, status);
        });
        PL_CHECK_LAUNCH("norm_rope_mix_write");
        return 0;
    }
    // Other sizes: a warp takes a head at a time, column by column; a block of four warps gets four head slots in
    // steps of few tokens (many small blocks fill the device) and eight in long steps (two a warp).
    const int heads_per_block = n_tokens >= 256 ? 8 : 4;
    const size_t smem = (static_cast<size_t>(rotary) + 32 + static_cast<size_t>(kThreads / 32) * dim) * sizeof(float);
    PL_REQUIRE(smem <= 48 * 1024, "norm_rope_mix_write: a key size of %d is too large", dim);
    const dim3 grid(n_tokens, (n_slots + heads_per_block - 1) / heads_per_block);
    PL_REQUIRE(grid.y <= 65535, "norm_rope_mix_write: too many heads (%d)", n_slots);
    PL_DISPATCH_DTYPE(dtype, "norm_rope_mix_write", {
        pl_launch_overlapped(norm_rope_mix_write_kernel<scalar_t>, grid, dim3(kThreads), smem, stream,
                             static_cast<const scalar_t*>(q), static_cast<const scalar_t*>(k),
                             static_cast<const scalar_t*>(v), row_stride, static_cast<const scalar_t*>(v_first),
                             v_first_stride, lambda, static_cast<scalar_t*>(q_out), pos, entry, table, table_width,
                             static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool), page_stride, head_stride,
                             page_size, n_pages, inv_freq, rotary, n_heads, n_kv, dim, vdim, row, heads_per_block, mode,
                             q_weight, k_weight, eps, status);
    });
    PL_CHECK_LAUNCH("norm_rope_mix_write");
    return 0;
}
