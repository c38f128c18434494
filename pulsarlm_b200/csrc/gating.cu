// Gates between matrix products: the gated activation of a feed-forward with a choice of
// activation, and an output gate per element.
//
//   gated_act:     out[t, i] = act(in[t, i]) * in[t, width + i]      act: silu or the tanh form of GELU
//   sigmoid_gate:  x[t, i]  *= sigmoid(gate[t, i])
//   sigmoid_gate_heads:  x[t, h, :] *= sigmoid(gate[t, h])     one gate per head
//
// Arithmetic in fp32 (expf, tanhf), one rounding on the store.
#include "common.cuh"

#include <algorithm>

namespace {

__device__ __forceinline__ float gate_activation(float z, int act) {
    if (act == 1) {
        // 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
        const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
        return 0.5f * z * (1.0f + tanhf(inner));
    }
    return z / (1.0f + expf(-z));
}

template <typename scalar_t>
__global__ void gated_act_kernel(const scalar_t* __restrict__ in, scalar_t* __restrict__ out, int64_t tokens,
                                 int width, int act) {
    pl_grid_trigger();
    pl_grid_wait();
    const int quads = width / 4;  // (the launcher takes this kernel for widths that are multiples of 4)
    const int64_t total = tokens * quads;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / quads;
        const int i = 4 * static_cast<int>(idx - t * quads);
        const float4 g = pl_load4(in + t * 2 * width + i);
        const float4 u = pl_load4(in + t * 2 * width + width + i);
        pl_store4(out + t * width + i, make_float4(gate_activation(g.x, act) * u.x, gate_activation(g.y, act) * u.y,
                                                   gate_activation(g.z, act) * u.z, gate_activation(g.w, act) * u.w));
    }
}

template <typename scalar_t>
__global__ void gated_act_scalar_kernel(const scalar_t* __restrict__ in, scalar_t* __restrict__ out, int64_t tokens,
                                        int width, int act) {
    pl_grid_trigger();
    pl_grid_wait();
    const int64_t total = tokens * width;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / width;
        const int i = static_cast<int>(idx - t * width);
        pl_store(out + idx, gate_activation(pl_load(in + t * 2 * width + i), act) * pl_load(in + t * 2 * width + width + i));
    }
}

template <typename scalar_t>
__global__ void sigmoid_gate_kernel(scalar_t* __restrict__ x, int64_t x_stride, const scalar_t* __restrict__ gate,
                                    int64_t gate_stride, int64_t tokens, int width) {
    pl_grid_trigger();
    pl_grid_wait();
    const int64_t total = tokens * width;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / width;
        const int i = static_cast<int>(idx - t * width);
        scalar_t* at = x + t * x_stride + i;
        pl_store(at, pl_load(at) / (1.0f + expf(-pl_load(gate + t * gate_stride + i))));
    }
}

// Four channels a thread, for widths, strides and addresses that are multiples of four elements.
template <typename scalar_t>
__global__ void sigmoid_gate_quads_kernel(scalar_t* __restrict__ x, int64_t x_stride, const scalar_t* __restrict__ gate,
                                          int64_t gate_stride, int64_t tokens, int width) {
    pl_grid_trigger();
    pl_grid_wait();
    const int quads = width / 4;
    const int64_t total = tokens * quads;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / quads;
        const int i = 4 * static_cast<int>(idx - t * quads);
        scalar_t* at = x + t * x_stride + i;
        const float4 v = pl_load4(at);
        const float4 g = pl_load4(gate + t * gate_stride + i);
        pl_store4(at, make_float4(v.x / (1.0f + expf(-g.x)), v.y / (1.0f + expf(-g.y)), v.z / (1.0f + expf(-g.z)),
                                  v.w / (1.0f + expf(-g.w))));
    }
}

// One gate per head: x [T, heads, row] times sigmoid(gate [T, heads]); PER elements a thread (1 or 4).
template <typename scalar_t, int PER>
__global__ void sigmoid_gate_heads_kernel(scalar_t* __restrict__ x, int64_t x_stride, const scalar_t* __restrict__ gate,
                                          int64_t gate_stride, int64_t tokens, int heads, int row) {
    pl_grid_trigger();
    pl_grid_wait();
    const int pieces = heads * row / PER;
    const int64_t total = tokens * pieces;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / pieces;
        const int i = PER * static_cast<int>(idx - t * pieces);
        const float factor = 1.0f / (1.0f + expf(-pl_load(gate + t * gate_stride + i / row)));
        scalar_t* at = x + t * x_stride + i;
        if (PER == 4) {
            const float4 v = pl_load4(at);
            pl_store4(at, make_float4(v.x * factor, v.y * factor, v.z * factor, v.w * factor));
        } else {
            pl_store(at, pl_load(at) * factor);
        }
    }
}

}  // namespace

// in [T, 2 * width] (gate columns, then up columns), out [T, width], both dense, in the
// engine's dtype. act 0: silu, 1: the tanh form of GELU.
PL_API int pl_gated_act(const void* in, void* out, int n_tokens, int width, int act, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0 && (act == 0 || act == 1), "gated_act: bad arguments tokens=%d width=%d "
               "act=%d", n_tokens, width, act);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = 256;
    const bool quads = width % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    const int64_t total = static_cast<int64_t>(n_tokens) * (quads ? width / 4 : width);
    const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
    PL_DISPATCH_DTYPE(dtype, "gated_act", {
        if (quads) {
            pl_launch_overlapped(gated_act_kernel<scalar_t>, dim3(blocks), dim3(threads), 0, stream,
                                 static_cast<const scalar_t*>(in), static_cast<scalar_t*>(out), n_tokens, width, act);
        } else {
            pl_launch_overlapped(gated_act_scalar_kernel<scalar_t>, dim3(blocks), dim3(threads), 0, stream,
                                 static_cast<const scalar_t*>(in), static_cast<scalar_t*>(out), n_tokens, width, act);
        }
    });
    PL_CHECK_LAUNCH("gated_act");
    return 0;
}

// x [T, width] (x_stride elements between rows) is multiplied in place by sigmoid(gate [T,
// width]) (gate_stride between rows), both in the engine's dtype.
PL_API int pl_sigmoid_gate(void* x, int64_t x_stride, const void* gate, int64_t gate_stride, int n_tokens, int width,
                           int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0, "sigmoid_gate: bad sizes tokens=%d width=%d", n_tokens, width);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = 256;
    const uintptr_t piece = dtype == PL_F32 ? 16 : 8;  // four elements
    const bool quads = width % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 &&
        reinterpret_cast<uintptr_t>(x) % piece == 0 && reinterpret_cast<uintptr_t>(gate) % piece == 0;
    const int64_t total = static_cast<int64_t>(n_tokens) * (quads ? width / 4 : width);
    const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
    PL_DISPATCH_DTYPE(dtype, "sigmoid_gate", {
        if (quads) {
            pl_launch_overlapped(sigmoid_gate_quads_kernel<scalar_t>, dim3(blocks), dim3(threads), 0, stream,
                                 static_cast<scalar_t*>(x), x_stride, static_cast<const scalar_t*>(gate), gate_stride,
                                 n_tokens, width);
            PL_CHECK_LAUNCH("sigmoid_gate");
            return 0;
        }
        pl_launch_overlapped(sigmoid_gate_kernel<scalar_t>, dim3(blocks), dim3(threads), 0, stream,
                             static_cast<scalar_t*>(x), x_stride, static_cast<const scalar_t*>(gate), gate_stride,
                             n_tokens, width);
    });
    PL_CHECK_LAUNCH("sigmoid_gate");
    return 0;
}

// x [T, n_heads, row] (x_stride elements between tokens) is multiplied in place by sigmoid(gate [T, n_heads])
// (gate_stride between rows), one gate per head, both in the engine's dtype.
PL_API int pl_sigmoid_gate_heads(void* x, int64_t x_stride, const void* gate, int64_t gate_stride, int n_tokens,
                                 int n_heads, int row, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && row > 0, "sigmoid_gate_heads: bad sizes tokens=%d heads=%d row=%d",
               n_tokens, n_heads, row);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = 256;
    const uintptr_t piece = dtype == PL_F32 ? 16 : 8;  // four elements
    const bool quads = row % 4 == 0 && x_stride % 4 == 0 && reinterpret_cast<uintptr_t>(x) % piece == 0;
    const int64_t total = static_cast<int64_t>(n_tokens) * n_heads * row / (quads ? 4 : 1);
    const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
    PL_DISPATCH_DTYPE(dtype, "sigmoid_gate_heads", {
        if (quads) {
            pl_launch_overlapped(sigmoid_gate_heads_kernel<scalar_t, 4>, dim3(blocks), dim3(threads), 0, stream,
                                 static_cast<scalar_t*>(x), x_stride, static_cast<const scalar_t*>(gate), gate_stride,
                                 n_tokens, n_heads, row);
        } else {
            pl_launch_overlapped(sigmoid_gate_heads_kernel<scalar_t, 1>, dim3(blocks), dim3(threads), 0, stream,
                                 static_cast<scalar_t*>(x), x_stride, static_cast<const scalar_t*>(gate), gate_stride,
                                 n_tokens, n_heads, row);
        }
    });
    PL_CHECK_LAUNCH("sigmoid_gate_heads");
    return 0;
}
