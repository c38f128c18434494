// A routed feed-forward (mixture of experts): the router, and the experts' products for
// steps of few tokens and for the float32 engine.
//
// Router (pl_moe_route), all fp32: logits z = W_r h, scores s = softmax(z) over all experts
// (or, `sigmoid_scores`, s = sigmoid(z) of each alone), choice scores c = s + correction.
// Experts form `n_groups` equal groups of neighbours; a group's score is the sum of its
// `group_top` largest choice scores (1: its largest), and only experts of the `keep` best
// groups can be chosen (the others count as minus infinity). The `top` largest choice scores
// are chosen (ties go to the lower index); their weights are their scores s (without the
// correction), with `renormalise` over the chosen scores' sum (+ 1e-20). One block per token.
//
// Experts (pl_moe_gate_up, pl_moe_down): expert e of a token computes W_down,e (silu(W_gate,e h)
// * (W_up,e h)); pl_moe_up takes the place of pl_moe_gate_up for experts without a gate, W_down,e
// act(W_up,e h) with act the square of relu. The first kernel takes a (token, chosen expert) pair per block row and writes
// the gated activation, a warp per feature (both rows of the feature read with 16-byte loads,
// the lanes' shares added in a fixed order); the second takes a token per block row and adds
// up its experts' down projections times their weights, plus an optional row that every
// token gets (a shared expert's output), a warp per output channel. Sums in fp32, one
// rounding on each store. A token's result depends on its own row only. These kernels read an
// expert's weights once per pair that chose it (from L2 when several pairs share an expert):
// right for steps of few tokens, where the weights' stream is what costs.
//
// pl_moe_sort: the (token, expert) pairs in expert order for the grouped products of long
// steps: counts per expert, their running sums, and for every pair its row in that order.
// One block.
#include "common.cuh"

namespace {

constexpr int kMaxGroupTop = 8;  // a group's score adds up at most this many of its experts' scores

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }

// Largest value and its lowest index over a warp.
__device__ __forceinline__ void warp_argmax(float& value, int& index) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other > value || (other == value && other_index < index)) {
            value = other;
            index = other_index;
        }
    }
}

template <typename scalar_t>
struct Vec;
template <>
struct Vec<float> {
    static constexpr int kCount = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <>
struct Vec<__nv_bfloat16> {
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
};

// TOKENS tokens per block (a long step reads the router's weights once per TOKENS tokens): the
// logits by a warp per expert for all of the block's tokens at once, then a warp per token
// chooses. A token's sums are the same whatever TOKENS is.
template <typename scalar_t, int TOKENS>
__global__ void __launch_bounds__(512, TOKENS > 1 ? 2 : 1) moe_route_kernel(const scalar_t* __restrict__ h, int64_t h_stride, const float* __restrict__ router,
                                 const float* __restrict__ correction, int32_t* __restrict__ ids,
                                 float* __restrict__ weights, int n_tokens, int hidden, int n_experts, int top,
                                 int n_groups, int keep, int sigmoid_scores, int group_top, int renormalise) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float shared[];
    float* rows = shared;                                   // [TOKENS][hidden]
    float* scores = rows + TOKENS * hidden;                 // [TOKENS][n_experts]  s
    float* choices = scores + TOKENS * n_experts;           // [TOKENS][n_experts]  s + correction, -inf once taken or shut out
    float* group_scores = choices + TOKENS * n_experts;     // [TOKENS][n_groups]
    const int t0 = blockIdx.x * TOKENS;
    const int here = min(TOKENS, n_tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    constexpr int kPer = Vec<scalar_t>::kCount;  // elements of a 16-byte load
    if (hidden % kPer == 0 && h_stride % kPer == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0) {
        // 16 bytes of a row per thread and turn, several turns' loads in flight
        const int per_row = hidden / kPer;
#pragma unroll 4
        for (int i = threadIdx.x; i < TOKENS * per_row; i += blockDim.x) {
            const int r = i / per_row, j = (i - r * per_row) * kPer;
            float x[kPer];
            if (r < here) {
                Vec<scalar_t>::load(h + static_cast<int64_t>(t0 + r) * h_stride + j, x);
            } else {
#pragma unroll
                for (int u = 0; u < kPer; ++u) {
                    x[u] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < kPer; u += 4) {
                *reinterpret_cast<float4*>(rows + r * hidden + j + u) = make_float4(x[u], x[u + 1], x[u + 2], x[u + 3]);
            }
        }
    } else {
        for (int i = threadIdx.x; i < TOKENS * hidden; i += blockDim.x) {
            const int r = i / hidden;
            rows[i] = r < here ? pl_load(h + static_cast<int64_t>(t0 + r) * h_stride + (i - r * hidden)) : 0.0f;
        }
    }
    __syncthreads();
    const bool vectors = (hidden & 3) == 0 && (reinterpret_cast<uintptr_t>(router) & 15) == 0;
    for (int e = warp; e < n_experts; e += warps) {
        const float* w = router + static_cast<int64_t>(e) * hidden;
        float z[TOKENS];
#pragma unroll
        for (int r = 0; r < TOKENS; ++r) {
            z[r] = 0.0f;
        }
        if (vectors) {
            // Eight of the lane's vectors of the expert's row are asked for before any is used (the row
            // comes from L2 or memory: one load at a time would make a chain of their latencies).
            constexpr int kAhead = TOKENS > 1 ? 4 : 8;
            for (int base = lane * 4; base < hidden; base += 128 * kAhead) {
                float4 wv[kAhead];
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const int i = base + 128 * u;
                    wv[u] = i < hidden ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const int i = base + 128 * u;
                    if (i < hidden) {
#pragma unroll
                        for (int r = 0; r < TOKENS; ++r) {
                            const float4 xv = *reinterpret_cast<const float4*>(rows + r * hidden + i);
                            z[r] = fmaf(xv.x, wv[u].x, z[r]);
                            z[r] = fmaf(xv.y, wv[u].y, z[r]);
                            z[r] = fmaf(xv.z, wv[u].z, z[r]);
                            z[r] = fmaf(xv.w, wv[u].w, z[r]);
                        }
                    }
                }
            }
        } else {
            for (int i = lane; i < hidden; i += 32) {
#pragma unroll
                for (int r = 0; r < TOKENS; ++r) {
                    z[r] = fmaf(rows[r * hidden + i], w[i], z[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < TOKENS; ++r) {
            const float total = pl_warp_sum(z[r]);
            if (lane == 0) {
                scores[r * n_experts + e] = total;
            }
        }
    }
    __syncthreads();
    if (warp >= here) {
        return;
    }
    const int t = t0 + warp;
    float* score = scores + warp * n_experts;
    float* choice = choices + warp * n_experts;
    float* group_score = group_scores + warp * n_groups;
    if (sigmoid_scores) {
        for (int e = lane; e < n_experts; e += 32) {
            const float s = 1.0f / (1.0f + expf(-score[e]));
            score[e] = s;
            choice[e] = s + (correction != nullptr ? correction[e] : 0.0f);
        }
    } else {
        float top_z = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) {
            top_z = fmaxf(top_z, score[e]);
        }
        top_z = pl_warp_max(top_z);
        float sum = 0.0f;
        for (int e = lane; e < n_experts; e += 32) {
            const float x = expf(score[e] - top_z);
            score[e] = x;
            sum += x;
        }
        sum = pl_warp_sum(sum);
        for (int e = lane; e < n_experts; e += 32) {
            const float s = score[e] / sum;
            score[e] = s;
            choice[e] = s + (correction != nullptr ? correction[e] : 0.0f);
        }
    }
    __syncwarp();
    const int per_group = n_experts / n_groups;
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            // the sum of the group's `group_top` largest choice scores (equal scores count once each)
            float total = 0.0f;
            int taken[kMaxGroupTop];
            for (int round = 0; round < min(group_top, per_group); ++round) {
                float best = -INFINITY;
                int index = -1;
                for (int j = 0; j < per_group; ++j) {
                    bool free = true;
                    for (int r = 0; r < round; ++r) {
                        free = free && taken[r] != j;
                    }
                    const float x = choice[g * per_group + j];
                    if (free && (index < 0 || x > best)) {
                        best = x;
                        index = j;
                    }
                }
                taken[round] = index;
                total += best;
            }
            group_score[g] = total;
        }
        __syncwarp();
        // The `keep` best groups stay (marked +inf as they are picked); the others are shut out.
        for (int round = 0; round < keep; ++round) {
            float value = -INFINITY;
            int index = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float x = group_score[g];
                if (x != INFINITY && (x > value || index == 0x7fffffff)) {
                    value = x;
                    index = g;
                }
            }
            warp_argmax(value, index);
            // (a lane with nothing left holds index 0x7fffffff and value -inf; equal values take the lower index)
            if (lane == 0 && index != 0x7fffffff) {
                group_score[index] = INFINITY;
            }
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32) {
            if (group_score[e / per_group] != INFINITY) {
                choice[e] = -INFINITY;
            }
        }
        __syncwarp();
    }
    float chosen_sum = 0.0f;
    for (int round = 0; round < top; ++round) {
        float value = -INFINITY;
        int index = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float x = choice[e];
            if (x > value) {
                value = x;
                index = e;
            }
        }
        warp_argmax(value, index);
        if (index == 0x7fffffff) {
            index = 0;  // (fewer open experts than `top`: cannot happen with sizes the launcher accepts)
        }
        if (lane == 0) {
            ids[static_cast<int64_t>(t) * top + round] = index;
            weights[static_cast<int64_t>(t) * top + round] = score[index];
            choice[index] = -INFINITY;
        }
        chosen_sum += score[index];
        __syncwarp();
    }
    if (renormalise) {
        const float inv = 1.0f / (chosen_sum + 1e-20f);
        for (int j = lane; j < top; j += 32) {
            weights[static_cast<int64_t>(t) * top + j] *= inv;
        }
    }
}

// Dot product of a weight row with an fp32 vector in shared memory over a warp: lane l takes
// the elements of vectors l, l + 32, ...; the lanes' sums are added as a tree.
template <typename scalar_t>
__device__ __forceinline__ float warp_dot(const scalar_t* __restrict__ w, const float* __restrict__ x, int n,
                                          bool vectors, int lane) {
    float sum = 0.0f;
    if (vectors) {
        constexpr int kCount = Vec<scalar_t>::kCount;
        for (int i = lane * kCount; i < n; i += 32 * kCount) {
            float wv[kCount];
            Vec<scalar_t>::load(w + i, wv);
#pragma unroll
            for (int j = 0; j < kCount; ++j) {
                sum = fmaf(wv[j], x[i + j], sum);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            sum = fmaf(pl_load(w + i), x[i], sum);
        }
    }
    return pl_warp_sum(sum);
}

// ROWS dot products at once, rows `row_stride` elements apart from `w`: every lane first asks for
// all the rows' vectors of its place, then multiplies, so that ROWS loads are in flight per lane.
template <typename scalar_t, int ROWS>
__device__ __forceinline__ void warp_dots(const scalar_t* __restrict__ w, int64_t row_stride,
                                          const float* __restrict__ x, int n, bool vectors, int lane,
                                          float (&sums)[ROWS]) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        sums[r] = 0.0f;
    }
    if (vectors) {
        constexpr int kCount = Vec<scalar_t>::kCount;
        for (int i = lane * kCount; i < n; i += 32 * kCount) {
            float wv[ROWS][kCount];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                Vec<scalar_t>::load(w + r * row_stride + i, wv[r]);
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
#pragma unroll
                for (int j = 0; j < kCount; ++j) {
                    sums[r] = fmaf(wv[r][j], x[i + j], sums[r]);
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                sums[r] = fmaf(pl_load(w + r * row_stride + i), x[i], sums[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        sums[r] = pl_warp_sum(sums[r]);
    }
}

// The same for two sets of rows against two vectors (two experts' rows for one token).
template <typename scalar_t, int ROWS>
__device__ __forceinline__ void warp_dots_two(const scalar_t* __restrict__ w0, const float* __restrict__ x0,
                                              const scalar_t* __restrict__ w1, const float* __restrict__ x1,
                                              int64_t row_stride, int n, bool vectors, int lane, float (&sums0)[ROWS],
                                              float (&sums1)[ROWS]) {
    if (!vectors) {
        warp_dots<scalar_t, ROWS>(w0, row_stride, x0, n, false, lane, sums0);
        warp_dots<scalar_t, ROWS>(w1, row_stride, x1, n, false, lane, sums1);
        return;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        sums0[r] = 0.0f;
        sums1[r] = 0.0f;
    }
    constexpr int kCount = Vec<scalar_t>::kCount;
    for (int i = lane * kCount; i < n; i += 32 * kCount) {
        float a[ROWS][kCount], b[ROWS][kCount];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            Vec<scalar_t>::load(w0 + r * row_stride + i, a[r]);
            Vec<scalar_t>::load(w1 + r * row_stride + i, b[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
#pragma unroll
            for (int j = 0; j < kCount; ++j) {
                sums0[r] = fmaf(a[r][j], x0[i + j], sums0[r]);
                sums1[r] = fmaf(b[r][j], x1[i + j], sums1[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        sums0[r] = pl_warp_sum(sums0[r]);
        sums1[r] = pl_warp_sum(sums1[r]);
    }
}

constexpr int kFeaturesPerWarp = 4;

// Block (pair, feature block): act[pair, f] = silu(gate_e[f] . h) * (up_e[f] . h).
template <typename scalar_t>
__global__ void moe_gate_up_kernel(const scalar_t* __restrict__ h, int64_t h_stride,
                                   const scalar_t* __restrict__ gate_up, const int32_t* __restrict__ ids,
                                   scalar_t* __restrict__ act, int hidden, int ff, int top, int n_experts,
                                   int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float row[];  // [hidden]
    const int pair = blockIdx.x;
    const int t = pair / top;
    const int e = ids[pair];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        row[i] = pl_load(h + t * h_stride + i);
    }
    __syncthreads();
    if (e < 0 || e >= n_experts) {
        return;
    }
    const scalar_t* weights = gate_up + static_cast<int64_t>(e) * 2 * ff * hidden;  // [gate rows; up rows]
    const int f0 = (blockIdx.y * warps + warp) * kFeaturesPerWarp;
    if (f0 + kFeaturesPerWarp <= ff) {
        // The warp's four gate rows are neighbours, and so are its up rows: eight loads in flight per lane.
        float g[kFeaturesPerWarp], u[kFeaturesPerWarp];
        warp_dots_two<scalar_t, kFeaturesPerWarp>(weights + static_cast<int64_t>(f0) * hidden, row,
                                                  weights + static_cast<int64_t>(ff + f0) * hidden, row, hidden, hidden,
                                                  vectors, lane, g, u);
        if (lane < kFeaturesPerWarp) {
            float gl = g[0], ul = u[0];
#pragma unroll
            for (int r = 1; r < kFeaturesPerWarp; ++r) {
                gl = lane == r ? g[r] : gl;
                ul = lane == r ? u[r] : ul;
            }
            pl_store(act + static_cast<int64_t>(pair) * ff + f0 + lane, silu_f32(gl) * ul);
        }
        return;
    }
    for (int f = f0; f < min(f0 + kFeaturesPerWarp, ff); ++f) {
        const float g = warp_dot<scalar_t>(weights + static_cast<int64_t>(f) * hidden, row, hidden, vectors, lane);
        const float u = warp_dot<scalar_t>(weights + static_cast<int64_t>(ff + f) * hidden, row, hidden, vectors, lane);
        if (lane == 0) {
            pl_store(act + static_cast<int64_t>(pair) * ff + f, silu_f32(g) * u);
        }
    }
}

// Block (pair, feature block): act[pair, f] = relu(up_e[f] . h)^2, for experts without a gate.
template <typename scalar_t>
__global__ void moe_up_kernel(const scalar_t* __restrict__ h, int64_t h_stride, const scalar_t* __restrict__ up,
                              const int32_t* __restrict__ ids, scalar_t* __restrict__ act, int hidden, int ff, int top,
                              int n_experts, int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float row[];  // [hidden]
    const int pair = blockIdx.x;
    const int t = pair / top;
    const int e = ids[pair];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        row[i] = pl_load(h + t * h_stride + i);
    }
    __syncthreads();
    if (e < 0 || e >= n_experts) {
        return;
    }
    const scalar_t* weights = up + static_cast<int64_t>(e) * ff * hidden;
    const int f0 = (blockIdx.y * warps + warp) * kFeaturesPerWarp;
    if (f0 + kFeaturesPerWarp <= ff) {
        float u[kFeaturesPerWarp];
        warp_dots<scalar_t, kFeaturesPerWarp>(weights + static_cast<int64_t>(f0) * hidden, hidden, row, hidden, vectors,
                                              lane, u);
        if (lane < kFeaturesPerWarp) {
            float ul = u[0];
#pragma unroll
            for (int r = 1; r < kFeaturesPerWarp; ++r) {
                ul = lane == r ? u[r] : ul;
            }
            ul = fmaxf(ul, 0.0f);
            pl_store(act + static_cast<int64_t>(pair) * ff + f0 + lane, ul * ul);
        }
        return;
    }
    for (int f = f0; f < min(f0 + kFeaturesPerWarp, ff); ++f) {
        float u = warp_dot<scalar_t>(weights + static_cast<int64_t>(f) * hidden, row, hidden, vectors, lane);
        if (lane == 0) {
            u = fmaxf(u, 0.0f);
            pl_store(act + static_cast<int64_t>(pair) * ff + f, u * u);
        }
    }
}

constexpr int kChannelsPerWarp = 4;

// Block (token, channel block): out[t, c] = sum_j weight[t, j] * (down_{e_j}[c] . act[t, j]) + also[t, c].
template <typename scalar_t>
__global__ void moe_down_kernel(const scalar_t* __restrict__ act, const scalar_t* __restrict__ down,
                                const int32_t* __restrict__ ids, const float* __restrict__ weights,
                                const scalar_t* __restrict__ also, scalar_t* __restrict__ out, int hidden, int ff,
                                int top, int n_experts, int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ float rows[];  // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) {
        rows[i] = pl_load(act + static_cast<int64_t>(t) * top * ff + i);
    }
    __syncthreads();
    const int c0 = (blockIdx.y * warps + warp) * kChannelsPerWarp;
    if (c0 + kChannelsPerWarp <= hidden) {
        float sums[kChannelsPerWarp];
#pragma unroll
        for (int r = 0; r < kChannelsPerWarp; ++r) {
            sums[r] = 0.0f;
        }
        // Two experts at a time: eight rows' loads in flight per lane. (The sums of an expert's rows are
        // made as for one expert alone, and added in the experts' order.)
        for (int j = 0; j < top; j += 2) {
            const int e0 = ids[static_cast<int64_t>(t) * top + j];
            const int e1 = j + 1 < top ? ids[static_cast<int64_t>(t) * top + j + 1] : -1;
            const bool ok0 = e0 >= 0 && e0 < n_experts, ok1 = e1 >= 0 && e1 < n_experts;
            float dots0[kChannelsPerWarp], dots1[kChannelsPerWarp];
            if (ok0 && ok1) {
                warp_dots_two<scalar_t, kChannelsPerWarp>(down + (static_cast<int64_t>(e0) * hidden + c0) * ff, rows + j * ff,
                                                          down + (static_cast<int64_t>(e1) * hidden + c0) * ff,
                                                          rows + (j + 1) * ff, ff, ff, vectors, lane, dots0, dots1);
            } else {
                if (ok0) {
                    warp_dots<scalar_t, kChannelsPerWarp>(down + (static_cast<int64_t>(e0) * hidden + c0) * ff, ff,
                                                          rows + j * ff, ff, vectors, lane, dots0);
                }
                if (ok1) {
                    warp_dots<scalar_t, kChannelsPerWarp>(down + (static_cast<int64_t>(e1) * hidden + c0) * ff, ff,
                                                          rows + (j + 1) * ff, ff, vectors, lane, dots1);
                }
            }
            if (ok0) {
                const float weight = weights[static_cast<int64_t>(t) * top + j];
#pragma unroll
                for (int r = 0; r < kChannelsPerWarp; ++r) {
                    sums[r] = fmaf(weight, dots0[r], sums[r]);
                }
            }
            if (ok1) {
                const float weight = weights[static_cast<int64_t>(t) * top + j + 1];
#pragma unroll
                for (int r = 0; r < kChannelsPerWarp; ++r) {
                    sums[r] = fmaf(weight, dots1[r], sums[r]);
                }
            }
        }
        if (lane < kChannelsPerWarp) {
            float sum = sums[0];
#pragma unroll
            for (int r = 1; r < kChannelsPerWarp; ++r) {
                sum = lane == r ? sums[r] : sum;
            }
            const int c = c0 + lane;
            if (also != nullptr) {
                sum += pl_load(also + static_cast<int64_t>(t) * hidden + c);
            }
            pl_store(out + static_cast<int64_t>(t) * hidden + c, sum);
        }
        return;
    }
    for (int c = c0; c < min(c0 + kChannelsPerWarp, hidden); ++c) {
        float sum = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int e = ids[static_cast<int64_t>(t) * top + j];
            if (e < 0 || e >= n_experts) {
                continue;
            }
            const scalar_t* w = down + (static_cast<int64_t>(e) * hidden + c) * ff;
            sum = fmaf(weights[static_cast<int64_t>(t) * top + j], warp_dot<scalar_t>(w, rows + j * ff, ff, vectors, lane),
                       sum);
        }
        if (lane == 0) {
            if (also != nullptr) {
                sum += pl_load(also + static_cast<int64_t>(t) * hidden + c);
            }
            pl_store(out + static_cast<int64_t>(t) * hidden + c, sum);
        }
    }
}

// One block: counts per expert (shared-memory atomics), their running sums, and each pair's row in
// expert order. The order of an expert's pairs among themselves is whatever the atomics give:
// a row's result in the grouped products does not depend on its place.
__global__ void moe_sort_kernel(const int32_t* __restrict__ ids, int n_pairs, int n_experts,
                                int32_t* __restrict__ ends, int32_t* __restrict__ row_of_pair,
                                int32_t* __restrict__ pair_of_row) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ int32_t starts[];  // [n_experts + 1] counts, then running sums; [n_experts] cursors
    int32_t* cursor = starts + n_experts + 1;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) {
        starts[e] = 0;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < n_experts) {
            atomicAdd(&starts[e + 1], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int e = 0; e < n_experts; ++e) {
            starts[e + 1] += starts[e];
            ends[e] = starts[e + 1];
            cursor[e] = starts[e];
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < n_experts) {
            const int at = atomicAdd(&cursor[e], 1);
            row_of_pair[p] = at;
            pair_of_row[at] = p;
        }
    }
}

// rows of x gathered into expert order: sorted[r] = x[pair_of_row[r] / top].
template <typename scalar_t>
__global__ void moe_gather_kernel(const scalar_t* __restrict__ x, int64_t x_stride,
                                  const int32_t* __restrict__ pair_of_row, scalar_t* __restrict__ sorted, int hidden,
                                  int top, int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    const int r = blockIdx.x;
    const int64_t t = pair_of_row[r] / top;
    constexpr int kPer = 16 / sizeof(scalar_t);
    if (vectors) {
        const uint4* from = reinterpret_cast<const uint4*>(x + t * x_stride);
        uint4* to = reinterpret_cast<uint4*>(sorted + static_cast<int64_t>(r) * hidden);
        for (int i = threadIdx.x; i < hidden / kPer; i += blockDim.x) {
            to[i] = from[i];
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        sorted[static_cast<int64_t>(r) * hidden + i] = x[t * x_stride + i];
    }
}

// out[t] = sum_j weight[t, j] * y[row_of_pair[t, j]] + also[t], fp32 sums, one rounding.
template <typename scalar_t>
__global__ void moe_combine_kernel(const scalar_t* __restrict__ y, const int32_t* __restrict__ row_of_pair,
                                   const float* __restrict__ weights, const scalar_t* __restrict__ also,
                                   scalar_t* __restrict__ out, int hidden, int top, int vectors) {
    pl_grid_trigger();
    pl_grid_wait();
    const int64_t t = blockIdx.x;
    if (vectors) {
        // (the same sums, four channels at a time)
        for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < top; ++j) {
                const float weight = weights[t * top + j];
                const float4 v = pl_load4(y + static_cast<int64_t>(row_of_pair[t * top + j]) * hidden + i);
                sum.x = fmaf(weight, v.x, sum.x);
                sum.y = fmaf(weight, v.y, sum.y);
                sum.z = fmaf(weight, v.z, sum.z);
                sum.w = fmaf(weight, v.w, sum.w);
            }
            if (also != nullptr) {
                const float4 v = pl_load4(also + t * hidden + i);
                sum.x += v.x;
                sum.y += v.y;
                sum.z += v.z;
                sum.w += v.w;
            }
            pl_store4(out + t * hidden + i, sum);
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float sum = 0.0f;
        for (int j = 0; j < top; ++j) {
            sum = fmaf(weights[t * top + j], pl_load(y + static_cast<int64_t>(row_of_pair[t * top + j]) * hidden + i), sum);
        }
        if (also != nullptr) {
            sum += pl_load(also + t * hidden + i);
        }
        pl_store(out + t * hidden + i, sum);
    }
}

}  // namespace

// h [T, hidden] (h_stride elements between rows) in the engine's dtype; router fp32 [n_experts,
// hidden]; correction fp32 [n_experts] or null; ids int32 [T, top]; weights fp32 [T, top].
// sigmoid_scores: s = sigmoid(z) instead of softmax(z); group_top: how many of a group's largest choice
// scores add up to its score; renormalise: whether the chosen scores are divided by their sum.
PL_API int pl_moe_route(const void* h, int64_t h_stride, const float* router, const float* correction, int32_t* ids,
                        float* weights, int n_tokens, int hidden, int n_experts, int top, int n_groups, int keep,
                        int sigmoid_scores, int group_top, int renormalise, int dtype, cudaStream_t stream) {
    PL_REQUIRE(group_top > 0 && group_top <= kMaxGroupTop, "moe_route: a group's score adds up 1 to %d scores, not %d",
               kMaxGroupTop, group_top);
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && n_experts > 0 && top > 0 && n_groups > 0 && keep > 0,
               "moe_route: bad sizes tokens=%d hidden=%d experts=%d top=%d groups=%d keep=%d", n_tokens, hidden,
               n_experts, top, n_groups, keep);
    PL_REQUIRE(n_experts % n_groups == 0 && keep <= n_groups, "moe_route: %d experts in %d groups of which %d stay",
               n_experts, n_groups, keep);
    PL_REQUIRE(top <= keep * (n_experts / n_groups), "moe_route: %d experts cannot be chosen from %d groups of %d", top,
               keep, n_experts / n_groups);
    const size_t per_token = (static_cast<size_t>(hidden) + 2 * n_experts + n_groups) * sizeof(float);
    PL_REQUIRE(per_token <= 200 * 1024, "moe_route: hidden %d and %d experts need too much shared memory", hidden,
               n_experts);
    if (n_tokens == 0) {
        return 0;
    }
    // Long steps take eight tokens per block when their rows fit (the width must be a multiple of 4
    // for the rows to stay on 16 bytes).
    const bool many = n_tokens >= 256 && 8 * per_token <= 200 * 1024 && hidden % 4 == 0;
    const size_t smem = (many ? 8 : 1) * per_token;
    const int threads = n_experts > 8 ? 512 : 256;
    PL_DISPATCH_DTYPE(dtype, "moe_route", {
        if (many) {
            if (smem > 48 * 1024) {
                cudaFuncSetAttribute(moe_route_kernel<scalar_t, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem));
            }
            // (room for two of these CTAs' rows per SM)
            cudaFuncSetAttribute(moe_route_kernel<scalar_t, 8>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
            pl_launch_overlapped(moe_route_kernel<scalar_t, 8>, dim3((n_tokens + 7) / 8), dim3(threads), smem, stream,
                                 static_cast<const scalar_t*>(h), h_stride, router, correction, ids, weights, n_tokens,
                                 hidden, n_experts, top, n_groups, keep, sigmoid_scores, group_top, renormalise);
        } else {
            if (smem > 48 * 1024) {
                cudaFuncSetAttribute(moe_route_kernel<scalar_t, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem));
            }
            pl_launch_overlapped(moe_route_kernel<scalar_t, 1>, dim3(n_tokens), dim3(threads), smem, stream,
                                 static_cast<const scalar_t*>(h), h_stride, router, correction, ids, weights, n_tokens,
                                 hidden, n_experts, top, n_groups, keep, sigmoid_scores, group_top, renormalise);
        }
    });
    PL_CHECK_LAUNCH("moe_route");
    return 0;
}

// gate_up [n_experts, 2 * ff, hidden] (an expert's gate rows, then its up rows); act [T * top, ff].
PL_API int pl_moe_gate_up(const void* h, int64_t h_stride, const void* gate_up, const int32_t* ids, void* act,
                          int n_tokens, int hidden, int ff, int top, int n_experts, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && ff > 0 && top > 0 && n_experts > 0, "moe_gate_up: bad sizes");
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    PL_REQUIRE(smem <= 200 * 1024, "moe_gate_up: hidden %d is too wide", hidden);
    if (n_tokens == 0) {
        return 0;
    }
    const int warps = 4;
    const dim3 grid(n_tokens * top, (ff + warps * kFeaturesPerWarp - 1) / (warps * kFeaturesPerWarp));
    PL_REQUIRE(grid.y <= 65535, "moe_gate_up: %d features per expert exceed the grid limit", ff);
    PL_DISPATCH_DTYPE(dtype, "moe_gate_up", {
        const int vectors = hidden % Vec<scalar_t>::kCount == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0;
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(moe_gate_up_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(moe_gate_up_kernel<scalar_t>, grid, dim3(warps * 32), smem, stream,
                             static_cast<const scalar_t*>(h), h_stride, static_cast<const scalar_t*>(gate_up), ids,
                             static_cast<scalar_t*>(act), hidden, ff, top, n_experts, vectors);
    });
    PL_CHECK_LAUNCH("moe_gate_up");
    return 0;
}

// up [n_experts, ff, hidden]; act [T * top, ff] = relu(up_e h)^2 for each pair's expert e.
PL_API int pl_moe_up(const void* h, int64_t h_stride, const void* up, const int32_t* ids, void* act, int n_tokens,
                     int hidden, int ff, int top, int n_experts, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && ff > 0 && top > 0 && n_experts > 0, "moe_up: bad sizes");
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    PL_REQUIRE(smem <= 200 * 1024, "moe_up: hidden %d is too wide", hidden);
    if (n_tokens == 0) {
        return 0;
    }
    const int warps = 4;
    const dim3 grid(n_tokens * top, (ff + warps * kFeaturesPerWarp - 1) / (warps * kFeaturesPerWarp));
    PL_REQUIRE(grid.y <= 65535, "moe_up: %d features per expert exceed the grid limit", ff);
    PL_DISPATCH_DTYPE(dtype, "moe_up", {
        const int vectors = hidden % Vec<scalar_t>::kCount == 0 && (reinterpret_cast<uintptr_t>(up) & 15) == 0;
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(moe_up_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(moe_up_kernel<scalar_t>, grid, dim3(warps * 32), smem, stream,
                             static_cast<const scalar_t*>(h), h_stride, static_cast<const scalar_t*>(up), ids,
                             static_cast<scalar_t*>(act), hidden, ff, top, n_experts, vectors);
    });
    PL_CHECK_LAUNCH("moe_up");
    return 0;
}

// act [T * top, ff]; down [n_experts, hidden, ff]; also [T, hidden] or null; out [T, hidden].
PL_API int pl_moe_down(const void* act, const void* down, const int32_t* ids, const float* weights, const void* also,
                       void* out, int n_tokens, int hidden, int ff, int top, int n_experts, int dtype,
                       cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && ff > 0 && top > 0 && n_experts > 0, "moe_down: bad sizes");
    const size_t smem = static_cast<size_t>(top) * ff * sizeof(float);
    PL_REQUIRE(smem <= 200 * 1024, "moe_down: %d experts of %d features need too much shared memory", top, ff);
    if (n_tokens == 0) {
        return 0;
    }
    const int warps = 4;
    const dim3 grid(n_tokens, (hidden + warps * kChannelsPerWarp - 1) / (warps * kChannelsPerWarp));
    PL_REQUIRE(grid.y <= 65535, "moe_down: hidden %d exceeds the grid limit", hidden);
    PL_DISPATCH_DTYPE(dtype, "moe_down", {
        const int vectors = ff % Vec<scalar_t>::kCount == 0 && (reinterpret_cast<uintptr_t>(down) & 15) == 0;
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(moe_down_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(moe_down_kernel<scalar_t>, grid, dim3(warps * 32), smem, stream,
                             static_cast<const scalar_t*>(act), static_cast<const scalar_t*>(down), ids, weights,
                             static_cast<const scalar_t*>(also), static_cast<scalar_t*>(out), hidden, ff, top,
                             n_experts, vectors);
    });
    PL_CHECK_LAUNCH("moe_down");
    return 0;
}

// ids int32 [n_pairs]; ends int32 [n_experts] (row after each expert's last); row_of_pair and
// pair_of_row int32 [n_pairs].
PL_API int pl_moe_sort(const int32_t* ids, int n_pairs, int n_experts, int32_t* ends, int32_t* row_of_pair,
                       int32_t* pair_of_row, cudaStream_t stream) {
    PL_REQUIRE(n_pairs >= 0 && n_experts > 0 && n_experts <= 8192, "moe_sort: bad sizes pairs=%d experts=%d", n_pairs,
               n_experts);
    const int threads = n_pairs >= 1024 ? 1024 : ((n_pairs + 31) / 32) * 32 > 32 ? ((n_pairs + 31) / 32) * 32 : 32;
    pl_launch_overlapped(moe_sort_kernel, dim3(1), dim3(threads), (2 * static_cast<size_t>(n_experts) + 1) * sizeof(int32_t),
                         stream, ids, n_pairs, n_experts, ends, row_of_pair, pair_of_row);
    PL_CHECK_LAUNCH("moe_sort");
    return 0;
}

PL_API int pl_moe_gather(const void* x, int64_t x_stride, const int32_t* pair_of_row, void* sorted, int n_pairs,
                         int hidden, int top, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_pairs >= 0 && hidden > 0 && top > 0, "moe_gather: bad sizes");
    if (n_pairs == 0) {
        return 0;
    }
    PL_DISPATCH_DTYPE(dtype, "moe_gather", {
        constexpr int kPer = 16 / sizeof(scalar_t);
        const int vectors = hidden % kPer == 0 && x_stride % kPer == 0 &&
            ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(sorted)) & 15) == 0;
        pl_launch_overlapped(moe_gather_kernel<scalar_t>, dim3(n_pairs), dim3(hidden >= 2048 ? 256 : 128), 0, stream,
                             static_cast<const scalar_t*>(x), x_stride, pair_of_row, static_cast<scalar_t*>(sorted),
                             hidden, top, vectors);
    });
    PL_CHECK_LAUNCH("moe_gather");
    return 0;
}

PL_API int pl_moe_combine(const void* y, const int32_t* row_of_pair, const float* weights, const void* also, void* out,
                          int n_tokens, int hidden, int top, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && top > 0, "moe_combine: bad sizes");
    if (n_tokens == 0) {
        return 0;
    }
    PL_DISPATCH_DTYPE(dtype, "moe_combine", {
        const int vectors = hidden % 4 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(also) |
                                                 reinterpret_cast<uintptr_t>(out)) & 15) == 0;
        pl_launch_overlapped(moe_combine_kernel<scalar_t>, dim3(n_tokens), dim3(hidden >= 1024 ? 256 : 128), 0, stream,
                             static_cast<const scalar_t*>(y), row_of_pair, weights, static_cast<const scalar_t*>(also),
                             static_cast<scalar_t*>(out), hidden, top, vectors);
    });
    PL_CHECK_LAUNCH("moe_combine");
    return 0;
}
