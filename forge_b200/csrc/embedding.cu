// Token embedding gather: out[t,:] = table[ids[t],:] * scale, written to the fp32 residual stream (or, with `add`, added to
// it: a design that feeds the embedding into the stream again before a repeated pass of its layers).
// Replaces the reference's embedding_kernel (src/operators/cuda/cuda_embedding.cu:9-34); like it,
// an id outside [0,V) gives a row of zeros, and here it also raises bit 0 of *status.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V, float scale, int add, int* status) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (!add) for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = (add ? o[c] : 0.f) + forge::to_float(row[c]) * scale;
}

// The same gather plus a row of a second table that the token and the token before it choose together:
//   row = (previous * mul_prev + current * mul_cur) mod buckets,   or row `buckets` (the table's last) at position 0.
// The token before the first token of a request's portion is the last token of its portion before, which is kept per
// request slot in `last` (int32, rows of `last_stride`).  The CTA of a request's first token of the step reads the kept
// token and then replaces it with the last token that the step brings for the request, so nobody else touches the slot.
template <typename T>
__global__ void embedding_pair_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ tok_req, const int32_t* __restrict__ q_start,
                                      const int32_t* __restrict__ slots, int32_t* __restrict__ last, long long last_stride,
                                      const T* __restrict__ table, const T* __restrict__ pair_table, float* __restrict__ out, int H,
                                      int V, int buckets, long long mul_prev, long long mul_cur, int* status) {
    __shared__ int s_prev;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t], s = tok_req[t];
    const bool first = t == q_start[s];
    if (threadIdx.x == 0) s_prev = first ? last[(size_t)slots[s] * last_stride] : ids[t - 1];
    __syncthreads();
    const int prev = s_prev;
    if (first && threadIdx.x == 0) last[(size_t)slots[s] * last_stride] = ids[q_start[s + 1] - 1];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V || (positions[t] > 0 && (prev < 0 || prev >= V))) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    long long row = buckets;
    if (positions[t] > 0) {
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const T* a = table + (size_t)id * H;
    const T* b = pair_table + (size_t)row * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = forge::to_float(a[c]) + forge::to_float(b[c]);
}

}  // namespace

// table [V, H] and pair_table [buckets + 1, H] of table_dtype; last int32 rows of last_stride (one per request slot).
extern "C" int forge_embedding_pair(const int32_t* ids, const int32_t* positions, const int32_t* tok_req, const int32_t* q_start,
                                    const int32_t* slots, int32_t* last, long long last_stride, const void* table,
                                    const void* pair_table, int table_dtype, float* out, int T, int H, int V, int buckets,
                                    long long mul_prev, long long mul_cur, int* status, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0 || buckets <= 0 || last_stride <= 0)
        return forge::fail(FORGE_ERR_ARG, "embedding_pair: bad sizes T=%d H=%d V=%d buckets=%d", T, H, V, buckets);
    if (T == 0) return FORGE_OK;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(table_dtype, TT,
        e = forge::launch(embedding_pair_kernel<TT>, dim3(T), dim3(threads), 0, stream, 1, ids, positions, tok_req, q_start, slots, last,
                          last_stride, (const TT*)table, (const TT*)pair_table, out, H, V, buckets, mul_prev, mul_cur, status));
    return forge::check_launch("embedding_pair", e);
}

extern "C" int forge_embedding(const int32_t* ids, const void* table, int table_dtype, float* out,
                               int T, int H, int V, float scale, int add, int* status, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return FORGE_OK;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(table_dtype, TT,
        e = forge::launch(embedding_kernel<TT>, dim3(T), dim3(threads), 0, stream, 1, ids, (const TT*)table, out, H, V, scale, add, status));
    return forge::check_launch("embedding", e);
}
