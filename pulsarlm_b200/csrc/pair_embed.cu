// An embedding with a second table indexed by a hash of (token before, token).
//
// x[t] = table[token[t]] + pairs[row(t)], written as fp32 into the residual stream, with
// row(t) = (before * mul_prev + token * mul_cur) mod buckets and, for the first token of a
// sequence (position 0), row(t) = buckets (the table's last row). The token before row t
// is the row above it when that belongs to the same entry of the step, else the last
// token of the request's earlier steps, which is kept in a state slot per request
// (int32 [slots, 1]). After the step the slot holds the entry's last token: in a step
// whose entries bring one token each the same launch writes it (the thread that read the
// slot), else a second small kernel does, so that no row reads a slot another row of the
// same launch is writing.
#include "common.cuh"

namespace {

template <typename scalar_t>
__global__ void pair_embed_kernel(const scalar_t* __restrict__ table, const scalar_t* __restrict__ pairs,
                                  const int32_t* __restrict__ tokens, const int32_t* __restrict__ pos,
                                  const int32_t* __restrict__ entry, const int32_t* __restrict__ slots,
                                  int32_t* __restrict__ last_token, float* __restrict__ x, int hidden, int vocab,
                                  int buckets, long long mul_prev, long long mul_cur, int single_tokens,
                                  int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();  // (a step's tokens may be written by the kernel before this one)
    const int t = blockIdx.x;
    int token = tokens[t];
    if (token < 0 || token >= vocab) {
        if (threadIdx.x == 0 && status != nullptr) {
            atomicOr(status, 1);
        }
        token = 0;
    }
    const int e = entry[t];
    int row = buckets;
    if (pos[t] > 0) {
        int before = t > 0 && entry[t - 1] == e ? tokens[t - 1] : last_token[slots[e]];
        before = min(max(before, 0), vocab - 1);
        long long hash = (static_cast<long long>(before) * mul_prev + static_cast<long long>(token) * mul_cur) % buckets;
        row = static_cast<int>(hash < 0 ? hash + buckets : hash);
    }
    const scalar_t* a = table + static_cast<int64_t>(token) * hidden;
    const scalar_t* b = pairs + static_cast<int64_t>(row) * hidden;
    float* out = x + static_cast<int64_t>(t) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        out[i] = pl_load(a + i) + pl_load(b + i);
    }
    if (single_tokens) {
        __syncthreads();  // (every thread has read the slot)
        if (threadIdx.x == 0) {
            last_token[slots[e]] = token;
        }
    }
}

__global__ void pair_embed_state_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ entry,
                                        const int32_t* __restrict__ slots, int32_t* __restrict__ last_token,
                                        int n_tokens) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_tokens && (t == n_tokens - 1 || entry[t + 1] != entry[t])) {
        last_token[slots[entry[t]]] = tokens[t];
    }
}

}  // namespace

// table [vocab, hidden] and pairs [buckets + 1, hidden] in the engine's dtype; tokens, pos, entry
// int32 [T]; slots int32 [entries]; last_token int32 [slots] (one per request slot); x fp32 [T,
// hidden]. single_tokens != 0: every entry of the step brings one token and the slots are moved on
// by the same launch; else pl_pair_embed_state must follow.
PL_API int pl_pair_embed(const void* table, const void* pairs, const int32_t* tokens, const int32_t* pos,
                         const int32_t* entry, const int32_t* slots, int32_t* last_token, float* x, int n_tokens,
                         int hidden, int vocab, int buckets, int64_t mul_prev, int64_t mul_cur, int single_tokens,
                         int dtype, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0 && buckets > 0,
               "pair_embed: bad sizes tokens=%d hidden=%d vocab=%d buckets=%d", n_tokens, hidden, vocab, buckets);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    PL_DISPATCH_DTYPE(dtype, "pair_embed", {
        pl_launch_overlapped(pair_embed_kernel<scalar_t>, dim3(n_tokens), dim3(threads), 0, stream,
                             static_cast<const scalar_t*>(table), static_cast<const scalar_t*>(pairs), tokens, pos,
                             entry, slots, last_token, x, hidden, vocab, buckets, static_cast<long long>(mul_prev),
                             static_cast<long long>(mul_cur), single_tokens, status);
    });
    PL_CHECK_LAUNCH("pair_embed");
    return 0;
}

PL_API int pl_pair_embed_state(const int32_t* tokens, const int32_t* entry, const int32_t* slots, int32_t* last_token,
                               int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) {
        return 0;
    }
    pl_launch_overlapped(pair_embed_state_kernel, dim3((n_tokens + 127) / 128), dim3(128), 0, stream, tokens, entry,
                         slots, last_token, n_tokens);
    PL_CHECK_LAUNCH("pair_embed_state");
    return 0;
}
