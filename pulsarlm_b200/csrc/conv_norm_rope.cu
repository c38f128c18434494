// What lies between the q/k projection and paged attention in a mixer whose values are its
// keys, in one pass over a token's row:
//
//   u[t]   = proj[t] + bias                                        q channels, then k channels
//   y[t]   = sum_j cw[:, j] * u[t - (taps - 1) + j]                 per channel; zeros before position 0
//   q^     = y_q * rsqrt(mean(y_q^2) + eps) * nq                    one norm over ALL q channels
//   k^     = y_k * rsqrt(mean(y_k^2) + eps) * nk                    one over all k channels
//   q, k   = rotate(q^), rotate(k^)                                per head, the first `rotary` columns
//   K page <- k,   V page <- y_k                                   the values are the filtered keys
//
// Earlier inputs of a sequence come from the step's own rows where the portion has them and
// from the request's state slot where not (the slot holds the last taps - 1 projected rows,
// without the bias, as the product wrote them); an input at a negative position is zero.
// In a step whose entries bring one token each (`update_state`) the slot moves on in the same
// launch; otherwise the caller updates it afterwards (short_conv.cu). Rotation: the angle
// pos * f_i is formed and reduced in fp64 (rope_helpers.cuh); `interleaved` pairs columns
// (2i, 2i + 1), otherwise (i, i + rotary / 2); cos and sin are multiplied by `amplitude`.
// Everything is fp32 with one rounding on each store; sums are added in an order fixed by
// the sizes alone. One block per token; the filtered row lives in shared memory.
#include "rope_helpers.cuh"

namespace {

template <typename scalar_t>
__global__ void conv_norm_rope_kernel(
        const scalar_t* __restrict__ proj, int64_t row_stride, const float* __restrict__ bias,
        const float* __restrict__ conv_weight, int taps, scalar_t* __restrict__ conv_state,
        const int32_t* __restrict__ slots, int update_state, const float* __restrict__ q_norm,
        const float* __restrict__ k_norm, float eps, const double* __restrict__ inv_freq, int rotary, int interleaved,
        float amplitude, const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
        const int32_t* __restrict__ table, int table_width, scalar_t* __restrict__ q_out, int64_t q_out_stride,
        scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool, int64_t page_stride, int64_t head_stride,
        int page_size, int n_pages, int n_heads, int n_kv, int head_dim, int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) float shared[];  // [q_width + k_width] filtered row, [rotary / 2] cos, sin
    __shared__ float scratch[32];
    const int q_width = n_heads * head_dim, k_width = n_kv * head_dim, width = q_width + k_width;
    float* row = shared;
    float* cosines = shared + width;
    float* sines = cosines + rotary / 2;
    const int t = blockIdx.x;
    const int e = entry[t];
    const int p = pos[t];
    const int reach = taps - 1;
    int inside = 0;  // rows before this one that belong to the same sequence (up to `reach`)
    while (inside < reach && t - inside - 1 >= 0 && entry[t - inside - 1] == e) {
        ++inside;
    }
    for (int i = threadIdx.x; i < rotary / 2; i += blockDim.x) {
        float c, s;
        rope_sincos(p, inv_freq[i], c, s);
        cosines[i] = c * amplitude;
        sines[i] = s * amplitude;
    }
    scalar_t* old = reach > 0 ? conv_state + static_cast<int64_t>(slots[e]) * reach * width : nullptr;
    float square_q = 0.0f, square_k = 0.0f;
    for (int ch = threadIdx.x; ch < width; ch += blockDim.x) {
        const float b = bias != nullptr ? bias[ch] : 0.0f;
        const scalar_t own = proj[static_cast<int64_t>(t) * row_stride + ch];
        float acc = 0.0f;
        for (int j = 0; j < reach; ++j) {
            const int back = reach - j;  // this tap reads the input `back` positions before
            float v = 0.0f;
            scalar_t stored;
            if (back <= inside) {
                stored = proj[static_cast<int64_t>(t - back) * row_stride + ch];
            } else {
                stored = old[static_cast<int64_t>(reach - (back - inside)) * width + ch];
            }
            if (p - back >= 0) {
                v = pl_load(&stored) + b;
            }
            acc = fmaf(conv_weight[static_cast<int64_t>(ch) * taps + j], v, acc);
            if (update_state && j > 0) {
                old[static_cast<int64_t>(j - 1) * width + ch] = stored;  // (inside == 0 here: `stored` is slot row j)
            }
        }
        if (update_state && reach > 0) {
            old[static_cast<int64_t>(reach - 1) * width + ch] = own;
        }
        const float last = conv_weight != nullptr ? conv_weight[static_cast<int64_t>(ch) * taps + reach] : 1.0f;
        acc = fmaf(last, pl_load(&own) + b, acc);
        row[ch] = acc;
        if (ch < q_width) {
            square_q += acc * acc;
        } else {
            square_k += acc * acc;
        }
    }
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_norm != nullptr) {
        inv_q = 1.0f / sqrtf(pl_block_sum(square_q, scratch) / static_cast<float>(q_width) + eps);
    }
    if (k_norm != nullptr) {
        inv_k = 1.0f / sqrtf(pl_block_sum(square_k, scratch) / static_cast<float>(k_width) + eps);
    }
    __syncthreads();
    const int page = table[static_cast<int64_t>(e) * table_width + p / page_size];
    const bool page_ok = page >= 0 && page < n_pages;
    if (!page_ok && threadIdx.x == 0 && status != nullptr && k_pool != nullptr) {
        atomicOr(status, 2);
    }
    const int half = rotary / 2;
    for (int ch = threadIdx.x; ch < width; ch += blockDim.x) {
        const bool is_q = ch < q_width;
        const int local = is_q ? ch : ch - q_width;
        const int head = local / head_dim, d = local - head * head_dim;
        const float* scale = is_q ? q_norm : k_norm;
        const float inv = is_q ? inv_q : inv_k;
        float value = row[ch] * inv * (scale != nullptr ? scale[local] : 1.0f);
        if (d < rotary) {
            int pair, partner;
            bool low;
            if (interleaved) {
                pair = d >> 1;
                partner = d ^ 1;
                low = (d & 1) == 0;
            } else {
                low = d < half;
                pair = low ? d : d - half;
                partner = low ? d + half : d - half;
            }
            const int other = ch - d + partner;
            const float mate = row[other] * inv * (scale != nullptr ? scale[other - (is_q ? 0 : q_width)] : 1.0f);
            value = low ? rope_lo(value, mate, cosines[pair], sines[pair]) : rope_hi(mate, value, cosines[pair], sines[pair]);
        }
        if (is_q) {
            pl_store(q_out + static_cast<int64_t>(t) * q_out_stride + ch, value);
        } else if (page_ok && k_pool != nullptr) {
            const int64_t at = page * page_stride + head * head_stride + static_cast<int64_t>(p % page_size) * head_dim + d;
            pl_store(k_pool + at, value);
            pl_store(v_pool + at, row[ch]);
        }
    }
}

// The rows a latent-attention layer caches and the rotated part of its queries:
//
//   c[t]      = z[t, :rank] * rsqrt(mean(z[t, :rank]^2) + eps) * weight      -> page row [0, rank)
//   shared[t] = rotate(z[t, rank : rank + rot])                              -> page row [rank, rank + rot)
//   q_out[t, h, rank : rank + rot] = rotate(q[t, h, dim : dim + rot])        for every head
//
// z may be nullptr (a layer that reads another layer's rows writes none). One block per token.
template <typename scalar_t>
__global__ void latent_rope_write_kernel(
        const scalar_t* __restrict__ q, int64_t q_stride, int n_heads, int dim, scalar_t* __restrict__ q_out,
        int64_t q_out_stride, const scalar_t* __restrict__ z, int64_t z_stride, const float* __restrict__ weight,
        float eps, int rank, int rot, const double* __restrict__ inv_freq, int interleaved, float amplitude,
        const int32_t* __restrict__ pos, const int32_t* __restrict__ entry, const int32_t* __restrict__ table,
        int table_width, scalar_t* __restrict__ pool, int64_t page_stride, int page_size, int n_pages,
        int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) float shared[];  // [rot / 2] cos, sin
    __shared__ float scratch[32];
    float* cosines = shared;
    float* sines = shared + rot / 2;
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c, s;
        rope_sincos(p, inv_freq[i], c, s);
        cosines[i] = c * amplitude;
        sines[i] = s * amplitude;
    }
    __syncthreads();
    auto turned = [&](const scalar_t* v, int d) -> float {
        int pair, partner;
        bool low;
        if (interleaved) {
            pair = d >> 1;
            partner = d ^ 1;
            low = (d & 1) == 0;
        } else {
            low = d < half;
            pair = low ? d : d - half;
            partner = low ? d + half : d - half;
        }
        const float value = pl_load(v + d), mate = pl_load(v + partner);
        return low ? rope_lo(value, mate, cosines[pair], sines[pair]) : rope_hi(mate, value, cosines[pair], sines[pair]);
    };
    const int row_size = rank + rot;
    for (int i = threadIdx.x; i < n_heads * rot; i += blockDim.x) {
        const int head = i / rot, d = i - head * rot;
        const scalar_t* v = q + static_cast<int64_t>(t) * q_stride + static_cast<int64_t>(head) * (dim + rot) + dim;
        pl_store(q_out + static_cast<int64_t>(t) * q_out_stride + static_cast<int64_t>(head) * row_size + rank + d,
                 turned(v, d));
    }
    if (z == nullptr) {
        return;
    }
    const scalar_t* zr = z + static_cast<int64_t>(t) * z_stride;
    float square = 0.0f;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        const float value = pl_load(zr + d);
        square += value * value;
    }
    const float inv = 1.0f / sqrtf(pl_block_sum(square, scratch) / static_cast<float>(rank) + eps);
    const int page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0 && status != nullptr) {
            atomicOr(status, 2);
        }
        return;
    }
    scalar_t* dst = pool + page * page_stride + static_cast<int64_t>(p % page_size) * row_size;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        pl_store(dst + d, pl_load(zr + d) * inv * weight[d]);
    }
    for (int d = threadIdx.x; d < rot; d += blockDim.x) {
        pl_store(dst + rank + d, turned(zr + rank, d));
    }
}

}  // namespace

// proj [T, >= (n_heads + n_kv) * head_dim] (q channels, then k channels; row_stride elements
// between rows), q_out [T, n_heads * head_dim] (q_out_stride between rows), conv_state [slots,
// taps - 1, (n_heads + n_kv) * head_dim] and the pools [pages, n_kv, page_size, head_dim] in the
// engine's dtype; bias, q_norm, k_norm (each may be nullptr) and conv_weight [channels, taps]
// (nullptr when taps == 1) fp32; inv_freq fp64 [rotary / 2] (nullptr when rotary == 0).
// update_state != 0: every entry brings one token and its slot moves on here. k_pool == nullptr:
// only q is made (a layer that reads another layer's cache).
PL_API int pl_conv_norm_rope_write(const void* proj, int64_t row_stride, const float* bias, const float* conv_weight,
                                   int taps, void* conv_state, const int32_t* slots, int update_state,
                                   const float* q_norm, const float* k_norm, float eps, const double* inv_freq,
                                   int rotary, int interleaved, float amplitude, const int32_t* pos,
                                   const int32_t* entry, const int32_t* table, int table_width, void* q_out,
                                   int64_t q_out_stride, void* k_pool, void* v_pool, int64_t page_stride,
                                   int64_t head_stride, int page_size, int n_pages, int n_tokens, int n_heads,
                                   int n_kv, int head_dim, int dtype, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv > 0 && head_dim > 0 && page_size > 0 && taps >= 1,
               "conv_norm_rope_write: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d page=%d taps=%d", n_tokens,
               n_heads, n_kv, head_dim, page_size, taps);
    PL_REQUIRE(rotary >= 0 && rotary % 2 == 0 && rotary <= head_dim, "conv_norm_rope_write: rotary=%d must be even "
               "and at most head_dim=%d", rotary, head_dim);
    PL_REQUIRE(rotary == 0 || inv_freq != nullptr, "conv_norm_rope_write: a rotation needs its frequencies");
    PL_REQUIRE(taps == 1 || (conv_weight != nullptr && conv_state != nullptr && slots != nullptr),
               "conv_norm_rope_write: a convolution needs its weights and state");
    const size_t smem = (static_cast<size_t>(n_heads + n_kv) * head_dim + rotary) * sizeof(float);
    PL_REQUIRE(smem <= 200 * 1024, "conv_norm_rope_write: %d channels exceed what a block's shared memory holds",
               (n_heads + n_kv) * head_dim);
    if (n_tokens == 0) {
        return 0;
    }
    PL_DISPATCH_DTYPE(dtype, "conv_norm_rope_write", {
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(conv_norm_rope_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(conv_norm_rope_kernel<scalar_t>, dim3(n_tokens), dim3(256), smem, stream,
                             static_cast<const scalar_t*>(proj), row_stride, bias, conv_weight, taps,
                             static_cast<scalar_t*>(conv_state), slots, update_state, q_norm, k_norm, eps, inv_freq,
                             rotary, interleaved, amplitude, pos, entry, table, table_width,
                             static_cast<scalar_t*>(q_out), q_out_stride, static_cast<scalar_t*>(k_pool),
                             static_cast<scalar_t*>(v_pool), page_stride, head_stride, page_size, n_pages, n_heads,
                             n_kv, head_dim, status);
    });
    PL_CHECK_LAUNCH("conv_norm_rope_write");
    return 0;
}

// q [T, n_heads, dim + rot] (q_stride elements between tokens), q_out [T, n_heads, rank + rot]
// (q_out_stride between tokens; only the last rot columns of every head are written), z [T,
// rank + rot] (z_stride between rows; nullptr: nothing is cached) and pool [pages, 1, page_size,
// rank + rot] in the engine's dtype; weight fp32 [rank]; inv_freq fp64 [rot / 2].
PL_API int pl_latent_rope_write(const void* q, int64_t q_stride, int n_heads, int dim, void* q_out,
                                int64_t q_out_stride, const void* z, int64_t z_stride, const float* weight, float eps,
                                int rank, int rot, const double* inv_freq, int interleaved, float amplitude,
                                const int32_t* pos, const int32_t* entry, const int32_t* table, int table_width,
                                void* pool, int64_t page_stride, int page_size, int n_pages, int n_tokens, int dtype,
                                int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && dim >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && page_size > 0,
               "latent_rope_write: bad sizes tokens=%d heads=%d dim=%d rank=%d rot=%d page=%d", n_tokens, n_heads, dim,
               rank, rot, page_size);
    PL_REQUIRE(rot == 0 || inv_freq != nullptr, "latent_rope_write: a rotation needs its frequencies");
    PL_REQUIRE(z == nullptr || (weight != nullptr && pool != nullptr), "latent_rope_write: rows to cache need the "
               "norm's weight and a pool");
    if (n_tokens == 0) {
        return 0;
    }
    const size_t smem = static_cast<size_t>(rot) * sizeof(float);
    PL_DISPATCH_DTYPE(dtype, "latent_rope_write", {
        pl_launch_overlapped(latent_rope_write_kernel<scalar_t>, dim3(n_tokens), dim3(128), smem, stream,
                             static_cast<const scalar_t*>(q), q_stride, n_heads, dim, static_cast<scalar_t*>(q_out),
                             q_out_stride, static_cast<const scalar_t*>(z), z_stride, weight, eps, rank, rot, inv_freq,
                             interleaved, amplitude, pos, entry, table, table_width, static_cast<scalar_t*>(pool),
                             page_stride, page_size, n_pages, status);
    });
    PL_CHECK_LAUNCH("latent_rope_write");
    return 0;
}
