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
    const int heads_per_block = n_tokens >= 64 ? n_slots : 4;
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
