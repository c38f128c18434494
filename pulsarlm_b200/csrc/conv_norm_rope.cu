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
#include <algorithm>
#include <cstdint>

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

// Sixteen bytes of a row at a time: eight bfloat16 or four float channels per thread.
template <typename scalar_t>
struct RowVec {
    static constexpr int kN = 16 / sizeof(scalar_t);
};
__device__ __forceinline__ void row_unpack(const uint4& raw, float (&o)[4]) {
    o[0] = __uint_as_float(raw.x);
    o[1] = __uint_as_float(raw.y);
    o[2] = __uint_as_float(raw.z);
    o[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void row_unpack(const uint4& raw, float (&o)[8]) {
    // (a bfloat16 is the upper half of a float: shifts and masks, no conversion unit)
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[2 * i] = __uint_as_float(words[i] << 16);
        o[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 row_pack(const float (&v)[4]) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
__device__ __forceinline__ uint4 row_pack(const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    }
    return raw;
}
template <int N>
__device__ __forceinline__ void row_floats(const float* p, float (&o)[N]) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        o[i] = v.x;
        o[i + 1] = v.y;
        o[i + 2] = v.z;
        o[i + 3] = v.w;
    }
}

// The same arithmetic, channel by channel, for shapes whose rows split into 16-byte pieces that
// stay inside a head (the launcher checks sizes, strides and addresses): a thread takes whole
// pieces, the taps are known to the compiler, a neighbouring pair of a rotation lies in one
// piece, both norms' sums go through one block reduction, and everything a token's place in
// the batch decides (its neighbours' entries, its slot, its page) is asked for at the start.
template <typename scalar_t, int TAPS, bool INTERLEAVED>
__global__ void conv_norm_rope_vec_kernel(
        const scalar_t* __restrict__ proj, int64_t row_stride, const float* __restrict__ bias,
        const float* __restrict__ conv_weight, scalar_t* __restrict__ conv_state,
        const int32_t* __restrict__ slots, int update_state, const float* __restrict__ q_norm,
        const float* __restrict__ k_norm, float eps, const double* __restrict__ inv_freq, int rotary,
        float amplitude, const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
        const int32_t* __restrict__ table, int table_width, scalar_t* __restrict__ q_out, int64_t q_out_stride,
        scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool, int64_t page_stride, int64_t head_stride,
        int page_size, int n_pages, int n_heads, int n_kv, int head_dim, int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    constexpr int N = RowVec<scalar_t>::kN;
    constexpr int kReach = TAPS - 1;
    extern __shared__ __align__(16) float shared[];  // [q_width + k_width] filtered row, [rotary / 2] cos, sin, [width / N]
    __shared__ float scratch[2];
    const int q_width = n_heads * head_dim, k_width = n_kv * head_dim, width = q_width + k_width;
    float* row = shared;
    float* cosines = shared + width;
    float* sines = cosines + rotary / 2;
    float* piece_squares = sines + rotary / 2;
    const int t = blockIdx.x;
    const int e = entry[t];
    const int p = pos[t];
    int before[kReach > 0 ? kReach : 1];
#pragma unroll
    for (int j = 0; j < kReach; ++j) {
        before[j] = t - 1 - j >= 0 ? entry[t - 1 - j] : -1;
    }
    const int page = table[static_cast<int64_t>(e) * table_width + p / page_size];
    scalar_t* old = kReach > 0 ? conv_state + static_cast<int64_t>(slots[e]) * kReach * width : nullptr;
    int inside = 0;  // rows before this one that belong to the same sequence (up to kReach)
#pragma unroll
    for (int j = 0; j < kReach; ++j) {
        inside += (inside == j && before[j] == e) ? 1 : 0;
    }
    for (int i = threadIdx.x; i < rotary / 2; i += blockDim.x) {
        float c, s;
        rope_sincos(p, inv_freq[i], c, s);
        cosines[i] = c * amplitude;
        sines[i] = s * amplitude;
    }
    for (int ch = threadIdx.x * N; ch < width; ch += blockDim.x * N) {
        float b[N], acc[N], v[N], w[N * TAPS];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            b[i] = 0.0f;
            acc[i] = 0.0f;
        }
        if (bias != nullptr) {
            row_floats<N>(bias + ch, b);
        }
        if (conv_weight != nullptr) {
            row_floats<N * TAPS>(conv_weight + static_cast<int64_t>(ch) * TAPS, w);
        } else {
#pragma unroll
            for (int i = 0; i < N * TAPS; ++i) {
                w[i] = 1.0f;
            }
        }
        const uint4 own = *reinterpret_cast<const uint4*>(proj + static_cast<int64_t>(t) * row_stride + ch);
        uint4 stored[kReach > 0 ? kReach : 1];
#pragma unroll
        for (int j = 0; j < kReach; ++j) {
            const int back = kReach - j;  // this tap reads the input `back` positions before
            const scalar_t* src = back <= inside ? proj + static_cast<int64_t>(t - back) * row_stride + ch
                                                 : old + static_cast<int64_t>(kReach - (back - inside)) * width + ch;
            stored[j] = *reinterpret_cast<const uint4*>(src);
        }
#pragma unroll
        for (int j = 0; j < kReach; ++j) {
            const int back = kReach - j;
            if (p - back >= 0) {
                row_unpack(stored[j], v);
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    acc[i] = fmaf(w[i * TAPS + j], v[i] + b[i], acc[i]);
                }
            }
            if (update_state && j > 0) {
                *reinterpret_cast<uint4*>(old + static_cast<int64_t>(j - 1) * width + ch) = stored[j];
            }
        }
        if (update_state && kReach > 0) {
            *reinterpret_cast<uint4*>(old + static_cast<int64_t>(kReach - 1) * width + ch) = own;
        }
        row_unpack(own, v);
        float squares = 0.0f;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            acc[i] = fmaf(w[i * TAPS + kReach], v[i] + b[i], acc[i]);
            squares = fmaf(acc[i], acc[i], squares);
        }
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            *reinterpret_cast<float4*>(row + ch + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        }
        piece_squares[ch / N] = squares;
    }
    // Both sums in an order that the sizes alone decide (not the block's size): the first warp adds
    // the pieces' sums, lane l those of pieces l, l + 32, ...
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x, q_pieces = q_width / N, pieces = width / N;
        float sum_q = 0.0f, sum_k = 0.0f;
        for (int i = lane; i < q_pieces; i += 32) {
            sum_q += piece_squares[i];
        }
        for (int i = q_pieces + lane; i < pieces; i += 32) {
            sum_k += piece_squares[i];
        }
        sum_q = pl_warp_sum(sum_q);
        sum_k = pl_warp_sum(sum_k);
        if (lane == 0) {
            scratch[0] = sum_q;
            scratch[1] = sum_k;
        }
    }
    __syncthreads();
    const float total_q = scratch[0], total_k = scratch[1];
    const float inv_q = q_norm != nullptr ? 1.0f / sqrtf(total_q / static_cast<float>(q_width) + eps) : 1.0f;
    const float inv_k = k_norm != nullptr ? 1.0f / sqrtf(total_k / static_cast<float>(k_width) + eps) : 1.0f;
    const bool page_ok = page >= 0 && page < n_pages;
    if (!page_ok && threadIdx.x == 0 && status != nullptr && k_pool != nullptr) {
        atomicOr(status, 2);
    }
    const int half = rotary / 2;
    for (int ch = threadIdx.x * N; ch < width; ch += blockDim.x * N) {
        const bool is_q = ch < q_width;
        const int local = is_q ? ch : ch - q_width;
        const int head = local / head_dim, d0 = local - head * head_dim;
        const float* scale = is_q ? q_norm : k_norm;
        const float inv = is_q ? inv_q : inv_k;
        float raw[N], g[N], value[N], turned[N];
        row_floats<N>(row + ch, raw);
        if (scale != nullptr) {
            row_floats<N>(scale + local, g);
        }
#pragma unroll
        for (int i = 0; i < N; ++i) {
            value[i] = raw[i] * inv * (scale != nullptr ? g[i] : 1.0f);
        }
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const int d = d0 + i;
            turned[i] = value[i];
            if (d < rotary) {
                if (INTERLEAVED) {
                    const int pair = d >> 1;
                    turned[i] = (i & 1) == 0 ? rope_lo(value[i], value[i ^ 1], cosines[pair], sines[pair])
                                             : rope_hi(value[i ^ 1], value[i], cosines[pair], sines[pair]);
                } else {
                    const bool low = d < half;
                    const int pair = low ? d : d - half;
                    const int other = ch - d0 + (low ? d + half : d - half);
                    const float mate = row[other] * inv * (scale != nullptr ? scale[other - (is_q ? 0 : q_width)] : 1.0f);
                    turned[i] = low ? rope_lo(value[i], mate, cosines[pair], sines[pair])
                                    : rope_hi(mate, value[i], cosines[pair], sines[pair]);
                }
            }
        }
        if (is_q) {
            *reinterpret_cast<uint4*>(q_out + static_cast<int64_t>(t) * q_out_stride + ch) = row_pack(turned);
        } else if (page_ok && k_pool != nullptr) {
            const int64_t at = page * page_stride + head * head_stride + static_cast<int64_t>(p % page_size) * head_dim + d0;
            *reinterpret_cast<uint4*>(k_pool + at) = row_pack(turned);
            *reinterpret_cast<uint4*>(v_pool + at) = row_pack(raw);
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

template <typename scalar_t, int TAPS, bool PAIRS>
void launch_conv_pieces_as(const void* proj, int64_t row_stride, const float* bias, const float* conv_weight,
                           void* conv_state, const int32_t* slots, int update_state, const float* q_norm,
                           const float* k_norm, float eps, const double* inv_freq, int rotary, float amplitude,
                           const int32_t* pos, const int32_t* entry, const int32_t* table, int table_width, void* q_out,
                           int64_t q_out_stride, void* k_pool, void* v_pool, int64_t page_stride, int64_t head_stride,
                           int page_size, int n_pages, int n_tokens, int n_heads, int n_kv, int head_dim,
                           int32_t* status, size_t smem, int threads, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(conv_norm_rope_vec_kernel<scalar_t, TAPS, PAIRS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    }
    pl_launch_overlapped(conv_norm_rope_vec_kernel<scalar_t, TAPS, PAIRS>, dim3(n_tokens), dim3(threads), smem, stream,
                         static_cast<const scalar_t*>(proj), row_stride, bias, conv_weight,
                         static_cast<scalar_t*>(conv_state), slots, update_state, q_norm, k_norm, eps, inv_freq, rotary,
                         amplitude, pos, entry, table, table_width, static_cast<scalar_t*>(q_out), q_out_stride,
                         static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool), page_stride, head_stride,
                         page_size, n_pages, n_heads, n_kv, head_dim, status);
}

// Launches the kernel of 16-byte pieces where the shape allows it; false where it does not.
template <typename scalar_t>
bool launch_conv_pieces(const void* proj, int64_t row_stride, const float* bias, const float* conv_weight, int taps,
                        void* conv_state, const int32_t* slots, int update_state, const float* q_norm,
                        const float* k_norm, float eps, const double* inv_freq, int rotary, int interleaved,
                        float amplitude, const int32_t* pos, const int32_t* entry, const int32_t* table,
                        int table_width, void* q_out, int64_t q_out_stride, void* k_pool, void* v_pool,
                        int64_t page_stride, int64_t head_stride, int page_size, int n_pages, int n_tokens, int n_heads,
                        int n_kv, int head_dim, int32_t* status, size_t smem, cudaStream_t stream) {
    constexpr int kN = RowVec<scalar_t>::kN;
    const int width = (n_heads + n_kv) * head_dim;
    auto whole = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    const bool pieces = taps <= 4 && head_dim % kN == 0 && row_stride % kN == 0 && q_out_stride % kN == 0 &&
                        page_stride % kN == 0 && head_stride % kN == 0 && whole(proj) && whole(q_out) && whole(k_pool) &&
                        whole(v_pool) && whole(conv_state) && whole(bias) && whole(conv_weight) && whole(q_norm) &&
                        whole(k_norm);
    if (!pieces) {
        return false;
    }
    const int threads = std::min(512, std::max(32, (width / kN + 31) / 32 * 32));  // a thread per piece, up to 512
    smem += static_cast<size_t>(width / kN) * sizeof(float);
    if (smem > 200 * 1024) {
        return false;
    }
#define PL_PIECES(TAPS)                                                                                              \
    if (interleaved) {                                                                                               \
        launch_conv_pieces_as<scalar_t, TAPS, true>(proj, row_stride, bias, conv_weight, conv_state, slots,          \
            update_state, q_norm, k_norm, eps, inv_freq, rotary, amplitude, pos, entry, table, table_width, q_out,   \
            q_out_stride, k_pool, v_pool, page_stride, head_stride, page_size, n_pages, n_tokens, n_heads, n_kv,     \
            head_dim, status, smem, threads, stream);                                                                \
    } else {                                                                                                         \
        launch_conv_pieces_as<scalar_t, TAPS, false>(proj, row_stride, bias, conv_weight, conv_state, slots,         \
            update_state, q_norm, k_norm, eps, inv_freq, rotary, amplitude, pos, entry, table, table_width, q_out,   \
            q_out_stride, k_pool, v_pool, page_stride, head_stride, page_size, n_pages, n_tokens, n_heads, n_kv,     \
            head_dim, status, smem, threads, stream);                                                                \
    }
    switch (taps) {
        case 1: PL_PIECES(1) break;
        case 2: PL_PIECES(2) break;
        case 3: PL_PIECES(3) break;
        default: PL_PIECES(4) break;
    }
#undef PL_PIECES
    return true;
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
        if (launch_conv_pieces<scalar_t>(proj, row_stride, bias, conv_weight, taps, conv_state, slots, update_state, q_norm,
                                         k_norm, eps, inv_freq, rotary, interleaved, amplitude, pos, entry, table,
                                         table_width, q_out, q_out_stride, k_pool, v_pool, page_stride, head_stride,
                                         page_size, n_pages, n_tokens, n_heads, n_kv, head_dim, status, smem, stream)) {
            PL_CHECK_LAUNCH("conv_norm_rope_write");
            return 0;
        }
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
