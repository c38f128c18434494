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
// Statistics, norm products, rotation and the mix are fp32, one rounding on each store. A
// block has 128 threads whatever the step, a head is summed by one warp and a whole projection
// by the block, so a token's sums are added in an order that only the sizes decide.
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
    static constexpr int kCount = 4;
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
    static constexpr int kCount = 8;
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

// The same for long steps: a block per token. The token's q | k | v columns (one stretch of the projection's
// output) come into shared memory as floats in one pass of 16-byte loads, every thread's loads in flight at
// once; the warps then work on their heads there and store whole 16-byte pieces. Every sum is added in the
// order of the kernel above (a head by a warp, lanes striding its columns; a whole projection by the block's
// 128 threads), so a token's bits do not depend on which of the two ran.
template <typename scalar_t>
__global__ void __launch_bounds__(kThreads)
norm_rope_mix_write_row_kernel(const scalar_t* __restrict__ proj, int64_t row_stride,
                               const scalar_t* __restrict__ v_first, int64_t v_first_stride, float lambda,
                               scalar_t* __restrict__ q_out, const int32_t* __restrict__ pos,
                               const int32_t* __restrict__ entry, const int32_t* __restrict__ table, int table_width,
                               scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool, int64_t page_stride,
                               int64_t head_stride, int page_size, int n_pages, const double* __restrict__ inv_freq,
                               int rotary, int n_heads, int n_kv, int dim, int vdim, int row, int mode,
                               const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                               int load_pieces, int store_pieces, int32_t* status) {
    extern __shared__ float shared[];  // [rotary] cos | sin, [32] scratch, the token's columns
    constexpr int kPer = Piece<scalar_t>::kCount;
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = shared;
    float* sn = shared + half;
    float* scratch = shared + rotary;
    float* cols = scratch + 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kThreads / 32;
    const int q_cols = n_heads * dim, k_cols = n_kv * dim, total = q_cols + k_cols + n_kv * vdim;
    const scalar_t* src = proj + t * row_stride;
    int done = 0;
    if (load_pieces) {
        done = total / kPer * kPer;
        for (int i = threadIdx.x * kPer; i < done; i += kThreads * kPer) {
            float piece[kPer];
            Piece<scalar_t>::load(src + i, piece);
#pragma unroll
            for (int u = 0; u < kPer; ++u) {
                cols[i + u] = piece[u];
            }
        }
    }
    for (int i = done + threadIdx.x; i < total; i += kThreads) {
        cols[i] = pl_load(src + i);
    }
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += kThreads) {
            rope_sincos(p, inv_freq[j], cs[j], sn[j]);
        }
    }
    int page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0 && status != nullptr) {
            atomicOr(status, 2);
        }
        page = -1;
    }
    __syncthreads();
    float whole_q = 1.0f, whole_k = 1.0f;
    if (mode == kWhole) {
        float sum = 0.0f;
        for (int i = threadIdx.x; i < q_cols; i += kThreads) {
            sum = fmaf(cols[i], cols[i], sum);
        }
        whole_q = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(q_cols) + eps);
        sum = 0.0f;
        for (int i = threadIdx.x; i < k_cols; i += kThreads) {
            sum = fmaf(cols[q_cols + i], cols[q_cols + i], sum);
        }
        whole_k = rsqrtf(pl_block_sum(sum, scratch) / static_cast<float>(k_cols) + eps);
    }
    const int n_slots = n_heads + 2 * n_kv;
    for (int slot = warp; slot < n_slots; slot += warps) {
        const bool is_v = slot >= n_heads + n_kv, is_q = slot < n_heads;
        if (!is_q && page < 0) {
            continue;
        }
        const int h = is_q ? slot : (is_v ? slot - n_heads - n_kv : slot - n_heads);
        const int own = is_v ? vdim : dim;
        float* buf = is_v ? cols + q_cols + k_cols + h * vdim : cols + slot * dim;
        float after = 1.0f;
        if (is_v) {
            if (v_first != nullptr) {
                const scalar_t* f = v_first + t * v_first_stride + static_cast<int64_t>(h) * vdim;
                for (int d = lane; d < vdim; d += 32) {
                    buf[d] = __fmaf_rn(lambda, pl_load(f + d), __fmul_rn(1.0f - lambda, buf[d]));
                }
            }
        } else {
            const float* weight = is_q ? q_weight : k_weight;
            if (weight != nullptr && mode == kWhole) {
                weight += static_cast<int64_t>(h) * dim;
            }
            float r = 1.0f;
            if (mode == kPerHead) {
                float sum = 0.0f;
                for (int d = lane; d < dim; d += 32) {
                    sum = fmaf(buf[d], buf[d], sum);
                }
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
            if (mode == kUnitAfter) {
                float sum2 = 0.0f;
                for (int d = lane; d < dim; d += 32) {
                    sum2 = fmaf(buf[d], buf[d], sum2);
                }
                after = rsqrtf(pl_warp_sum(sum2) / static_cast<float>(dim) + eps);
            }
        }
        __syncwarp();
        scalar_t* to = is_q ? q_out + (static_cast<int64_t>(t) * n_heads + h) * row
                            : (is_v ? v_pool : k_pool) + page * page_stride + h * head_stride +
                                  static_cast<int64_t>(p % page_size) * row;
        if (store_pieces) {
            for (int d0 = lane * kPer; d0 < row; d0 += 32 * kPer) {
                float piece[kPer];
#pragma unroll
                for (int u = 0; u < kPer; ++u) {
                    piece[u] = d0 + u < own ? buf[d0 + u] * after : 0.0f;
                }
                Piece<scalar_t>::store(to + d0, piece);
            }
        } else {
            for (int d = lane; d < row; d += 32) {
                pl_store(to + d, d < own ? buf[d] * after : 0.0f);
            }
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
    // Long steps whose q, k and v are one stretch of the projection's output: a block per token that brings the
    // stretch into shared memory first (16-byte loads and stores where the addresses allow).
    const size_t elem = dtype == PL_F32 ? 4 : 2;
    const int64_t q_cols = static_cast<int64_t>(n_heads) * dim, k_cols = static_cast<int64_t>(n_kv) * dim;
    const size_t row_smem = (static_cast<size_t>(rotary) + 32 + q_cols + k_cols + static_cast<size_t>(n_kv) * vdim) * sizeof(float);
    const bool one_stretch = static_cast<const char*>(k) == static_cast<const char*>(q) + q_cols * elem &&
        static_cast<const char*>(v) == static_cast<const char*>(k) + k_cols * elem;
    if (n_tokens >= 256 && one_stretch && row_smem <= 160 * 1024) {
        const int per = static_cast<int>(16 / elem);
        const auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
        const int load_pieces = aligned(q) && row_stride % per == 0;
        const int store_pieces = row % per == 0 && aligned(q_out) && aligned(k_pool) && aligned(v_pool) &&
            page_stride % per == 0 && head_stride % per == 0;
        PL_DISPATCH_DTYPE(dtype, "norm_rope_mix_write", {
            if (row_smem > 48 * 1024) {
                cudaFuncSetAttribute(norm_rope_mix_write_row_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(row_smem));
            }
            pl_launch_overlapped(norm_rope_mix_write_row_kernel<scalar_t>, dim3(n_tokens), dim3(kThreads), row_smem, stream,
                                 static_cast<const scalar_t*>(q), row_stride, static_cast<const scalar_t*>(v_first),
                                 v_first_stride, lambda, static_cast<scalar_t*>(q_out), pos, entry, table, table_width,
                                 static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool), page_stride, head_stride,
                                 page_size, n_pages, inv_freq, rotary, n_heads, n_kv, dim, vdim, row, mode, q_weight,
                                 k_weight, eps, load_pieces, store_pieces, status);
        });
        PL_CHECK_LAUNCH("norm_rope_mix_write");
        return 0;
    }
    // Else a warp takes a head at a time: a block of four warps gets four head slots in steps of few tokens (many
    // small blocks fill the device) and eight in long steps (two a warp).
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
