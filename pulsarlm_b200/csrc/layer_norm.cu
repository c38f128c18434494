// Layer norm (weight and bias) on a sublayer's output as it enters the residual stream,
// fused with whatever reads the stream next:
//
//   u   = y                                                     the sublayer's output (optional)
//   v   = x + (u - mean(u)) / sqrt(var(u) + eps_y) * wy + by     into the fp32 residual stream
//   out = v                                                     rounded to the engine's dtype, or
//   out = (v - mean(v)) / sqrt(var(v) + eps) * w + b            the model's last norm
//
// var is the mean of the squared deviations, formed in a second pass over the row. One
// block per row, the row kept in shared memory. Statistics and the residual sum are fp32
// and added in an order that depends on the width alone, so a row's result does not depend
// on what else is in the batch.
#include <algorithm>
#include <cstdint>

#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void add_layernorm_kernel(float* __restrict__ x, const scalar_t* __restrict__ y,
                                     const float* __restrict__ wy, const float* __restrict__ by, float eps_y,
                                     scalar_t* __restrict__ out, const float* __restrict__ w,
                                     const float* __restrict__ b, float eps, const int32_t* __restrict__ rows,
                                     int hidden, int norm_out) {
    pl_grid_trigger();
    pl_grid_wait();
    extern __shared__ __align__(16) float row_values[];  // [hidden]: u, then v
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const float n = static_cast<float>(hidden);
    if (y != nullptr) {
        const scalar_t* yr = y + s * hidden;
        float local = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float u = pl_load(yr + i);
            row_values[i] = u;
            local += u;
        }
        const float mean = pl_block_sum(local, scratch) / n;
        local = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float d = row_values[i] - mean;
            local += d * d;
        }
        const float inv = 1.0f / sqrtf(pl_block_sum(local, scratch) / n + eps_y);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = xr[i] + ((row_values[i] - mean) * inv * wy[i] + by[i]);
            row_values[i] = v;
            if (rows == nullptr) {
                xr[i] = v;
            }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            row_values[i] = xr[i];
        }
    }
    if (out == nullptr) {
        return;
    }
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    if (!norm_out) {
        // (every thread reads back only what it wrote itself)
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            pl_store(outr + i, row_values[i]);
        }
        return;
    }
    float local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        local += row_values[i];
    }
    const float mean = pl_block_sum(local, scratch) / n;
    local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_values[i] - mean;
        local += d * d;
    }
    const float inv = 1.0f / sqrtf(pl_block_sum(local, scratch) / n + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        pl_store(outr + i, (row_values[i] - mean) * inv * w[i] + b[i]);
    }
}

// The same for widths that are a multiple of four and at most 4 * PER * blockDim: a thread keeps
// its PER groups of four channels in registers from the first load to the last store, and every
// load that does not wait for a statistic (the stream's row, the weights) is issued before the
// first reduction.
template <typename scalar_t, int PER>
__global__ void add_layernorm_vec_kernel(float* __restrict__ x, const scalar_t* __restrict__ y,
                                         const float* __restrict__ wy, const float* __restrict__ by, float eps_y,
                                         scalar_t* __restrict__ out, const float* __restrict__ w,
                                         const float* __restrict__ b, float eps, const int32_t* __restrict__ rows,
                                         int hidden, int norm_out) {
    pl_grid_trigger();
    pl_grid_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const float n = static_cast<float>(hidden);
    float4 v[PER];
    bool mine[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        mine[k] = i < hidden;
        v[k] = mine[k] ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    auto sum_of = [&](const float4 (&q)[PER]) {
        float local = 0.0f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            local += (q[k].x + q[k].y) + (q[k].z + q[k].w);  // (groups that are not this thread's hold zeros)
        }
        return pl_block_sum(local, scratch);
    };
    auto squares_of = [&](const float4 (&q)[PER], float mean) {
        float local = 0.0f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (mine[k]) {
                const float dx = q[k].x - mean, dy = q[k].y - mean, dz = q[k].z - mean, dw = q[k].w - mean;
                local += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
        return pl_block_sum(local, scratch);
    };
    if (y != nullptr) {
        const scalar_t* yr = y + s * hidden;
        float4 u[PER], g[PER], o[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 4;
            const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            u[k] = mine[k] ? pl_load4(yr + i) : zero;
            g[k] = mine[k] ? *reinterpret_cast<const float4*>(wy + i) : zero;
            o[k] = mine[k] ? *reinterpret_cast<const float4*>(by + i) : zero;
        }
        const float mean = sum_of(u) / n;
        const float inv = 1.0f / sqrtf(squares_of(u, mean) / n + eps_y);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (mine[k]) {
                v[k].x = v[k].x + ((u[k].x - mean) * inv * g[k].x + o[k].x);
                v[k].y = v[k].y + ((u[k].y - mean) * inv * g[k].y + o[k].y);
                v[k].z = v[k].z + ((u[k].z - mean) * inv * g[k].z + o[k].z);
                v[k].w = v[k].w + ((u[k].w - mean) * inv * g[k].w + o[k].w);
                if (rows == nullptr) {
                    *reinterpret_cast<float4*>(xr + (threadIdx.x + k * blockDim.x) * 4) = v[k];
                }
            }
        }
    }
    if (out == nullptr) {
        return;
    }
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    if (!norm_out) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (mine[k]) {
                pl_store4(outr + (threadIdx.x + k * blockDim.x) * 4, v[k]);
            }
        }
        return;
    }
    float4 g[PER], o[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        g[k] = mine[k] ? *reinterpret_cast<const float4*>(w + i) : zero;
        o[k] = mine[k] ? *reinterpret_cast<const float4*>(b + i) : zero;
    }
    const float mean = sum_of(v) / n;
    const float inv = 1.0f / sqrtf(squares_of(v, mean) / n + eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        if (mine[k]) {
            pl_store4(outr + (threadIdx.x + k * blockDim.x) * 4,
                      make_float4((v[k].x - mean) * inv * g[k].x + o[k].x, (v[k].y - mean) * inv * g[k].y + o[k].y,
                                  (v[k].z - mean) * inv * g[k].z + o[k].z, (v[k].w - mean) * inv * g[k].w + o[k].w));
        }
    }
}

template <typename scalar_t, int PER>
void launch_add_layernorm_vec(float* x, const void* y, const float* wy, const float* by, float eps_y, void* out,
                              const float* w, const float* b, float eps, const int32_t* rows, int n_rows, int hidden,
                              int norm_out, cudaStream_t stream) {
    const int threads = std::max(32, ((hidden / 4 + PER - 1) / PER + 31) / 32 * 32);
    pl_launch_overlapped(add_layernorm_vec_kernel<scalar_t, PER>, dim3(n_rows), dim3(threads), 0, stream, x,
                         static_cast<const scalar_t*>(y), wy, by, eps_y, static_cast<scalar_t*>(out), w, b, eps, rows,
                         hidden, norm_out);
}

}  // namespace

// x fp32 [T, hidden] (updated in place unless `rows` is given); y [T, hidden] in the engine's
// dtype or nullptr (nothing pending); wy, by, w, b fp32 [hidden]; out [n_rows, hidden] in the
// engine's dtype or nullptr. norm_out = 0: out is the stream rounded; 1: its layer norm with
// w, b, eps. With rows (int32 [n_rows]) output row r is made from source row rows[r] and x
// is left as it was.
PL_API int pl_add_layernorm(float* x, const void* y, const float* wy, const float* by, float eps_y, void* out,
                            const float* w, const float* b, float eps, const int32_t* rows, int n_rows, int hidden,
                            int norm_out, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_rows >= 0 && hidden > 0, "add_layernorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    PL_REQUIRE(y == nullptr || (wy != nullptr && by != nullptr), "add_layernorm: a pending output needs its norm's "
               "weight and bias");
    PL_REQUIRE(!norm_out || out == nullptr || (w != nullptr && b != nullptr), "add_layernorm: the output's norm "
               "needs a weight and a bias");
    PL_REQUIRE(static_cast<size_t>(hidden) * sizeof(float) <= 200 * 1024, "add_layernorm: hidden=%d exceeds what a "
               "block's shared memory holds", hidden);
    if (n_rows == 0) {
        return 0;
    }
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    auto whole = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    const bool groups = hidden % 4 == 0 && hidden <= 8192 && whole(x) && whole(y) && whole(wy) && whole(by) &&
                        whole(out) && whole(w) && whole(b);
    PL_DISPATCH_DTYPE(dtype, "add_layernorm", {
        if (groups) {
            if (hidden <= 2048) {
                launch_add_layernorm_vec<scalar_t, 1>(x, y, wy, by, eps_y, out, w, b, eps, rows, n_rows, hidden, norm_out,
                                                      stream);
            } else if (hidden <= 4096) {
                launch_add_layernorm_vec<scalar_t, 2>(x, y, wy, by, eps_y, out, w, b, eps, rows, n_rows, hidden, norm_out,
                                                      stream);
            } else {
                launch_add_layernorm_vec<scalar_t, 4>(x, y, wy, by, eps_y, out, w, b, eps, rows, n_rows, hidden, norm_out,
                                                      stream);
            }
            PL_CHECK_LAUNCH("add_layernorm");
            return 0;
        }
        if (smem > 48 * 1024) {
            cudaFuncSetAttribute(add_layernorm_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        }
        pl_launch_overlapped(add_layernorm_kernel<scalar_t>, dim3(n_rows), dim3(threads), smem, stream, x,
                             static_cast<const scalar_t*>(y), wy, by, eps_y, static_cast<scalar_t*>(out), w, b, eps,
                             rows, hidden, norm_out);
    });
    PL_CHECK_LAUNCH("add_layernorm");
    return 0;
}
