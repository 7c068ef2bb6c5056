// Small row-wise steps on the float32 residual stream that sit between a model's layers:
//   * an embedding with a second table indexed by a hash of (previous token, token), the previous
//     token of a request's first row of a step coming from per-request state;
//   * the start of a pass over a stretch of layers: a saved copy of the stream and / or one
//     vector are added to every row;
//   * a per-token side input: gelu_tanh(a) times a slice of a table row chosen by the token, and the
//     add of its projection, divided by its root mean square and weighted, to the stream;
//   * the stream rounded to the activation dtype for a product that reads it.
// One block per row; everything is float32 arithmetic.
#include "common.cuh"

using namespace cj;

namespace {

// out[t] = table[id] + pair[row], row = (prev * mul_prev + id * mul_cur) mod buckets, or row
// `buckets` for a request's first token (position 0).  prev is the token of row t - 1 when that
// row belongs to the same request, else the request's entry in `state` (its last token of the
// step before).
template <typename TW>
__global__ void pair_embed_kernel(float* __restrict__ out, const TW* __restrict__ table, const TW* __restrict__ pair,
                                  const int* __restrict__ ids, const int* __restrict__ positions,
                                  const int* __restrict__ row_req, const int* __restrict__ req_start,
                                  const int* __restrict__ req_slot, const int* __restrict__ state, int H, int V,
                                  int buckets, long long mul_prev, long long mul_cur) {
    cj::after_predecessor();
    cj::release_successor();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;                 // the host checks ids; an id out of range reads nothing
    int row = buckets;
    if (positions[t] > 0) {
        const int r = row_req[t];
        int prev = t > req_start[r] ? ids[t - 1] : state[req_slot[r]];
        row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets);
    }
    const TW* a = table + (size_t)(ok ? id : 0) * H;
    const TW* b = pair + (size_t)row * H;
    float* dst = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? to_f32(a[i]) + to_f32(b[i]) : 0.0f;
}

// after pair_embed: every request's last token of the step becomes its state (requests that a
// step's layout is filled up with have no rows and slot -1)
__global__ void pair_commit_kernel(const int* __restrict__ ids, const int* __restrict__ req_start,
                                   const int* __restrict__ req_slot, int* __restrict__ state, int requests) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= requests) return;
    const int lo = req_start[r], hi = req_start[r + 1], slot = req_slot[r];
    if (hi > lo && slot >= 0) state[slot] = ids[hi - 1];
}

// hs[t] += (other ? other[t] : 0) + (vec ? vec : 0)
__global__ void add_rows_kernel(float* __restrict__ hs, const float* __restrict__ other, const float* __restrict__ vec, int H) {
    cj::after_predecessor();
    cj::release_successor();
    const size_t base = (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hs[base + i];
        if (other) v += other[base + i];
        if (vec) v += vec[i];
        hs[base + i] = v;
    }
}

// hs[i] += parts[0][i] + parts[1][i] + ... in that order (partial sums of a product cut along K)
template <bool VEC>
__global__ void add_partials_kernel(float* __restrict__ hs, const float* __restrict__ parts, int n_parts, long long stride, long long n) {
    cj::after_predecessor();
    cj::release_successor();
    constexpr int W = VEC ? 4 : 1;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * W; i < n; i += (long long)gridDim.x * blockDim.x * W) {
        if (VEC) {
            float4 v = *(const float4*)(hs + i);
            for (int s = 0; s < n_parts; ++s) {
                const float4 p = *(const float4*)(parts + s * stride + i);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            *(float4*)(hs + i) = v;
        } else {
            float v = hs[i];
            for (int s = 0; s < n_parts; ++s) v += parts[s * stride + i];
            hs[i] = v;
        }
    }
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], offset + j]
template <typename TW, typename TO>
__global__ void gelu_gate_kernel(const float* __restrict__ a, int lda, const TW* __restrict__ table, int ldt, int offset,
                                 const int* __restrict__ ids, int V, TO* __restrict__ out, int n) {
    cj::after_predecessor();
    cj::release_successor();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    const TW* e = table + (size_t)(ok ? id : 0) * ldt + offset;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
        out[(size_t)t * n + j] = from_f32<TO>(ok ? gelu_tanh(a[(size_t)t * lda + j]) * to_f32(e[j]) : 0.0f);
}

// out = x in out's type
template <typename TO>
__global__ void cast_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    cj::after_predecessor();
    cj::release_successor();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(x[i]);
}

// hs[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w
__global__ void __launch_bounds__(256) norm_add_kernel(float* __restrict__ hs, const float* __restrict__ y,
                                                       const float* __restrict__ w, float eps, int H) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float part[8];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(y[base + i], y[base + i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += part[i];
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) hs[base + i] += y[base + i] * inv * w[i];
}

}  // namespace

CJ_EXPORT int cj_stream_cast(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!x || !out) return CJ_ERR_ARG;
    long long blocks = (n + 1023) / 1024;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == CJ_BF16) cj::launch(cast_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, n);
    else if (out_dtype == CJ_F32) cj::launch(cast_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (float*)out, n);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_stream_norm_add(float* hs, const float* y, const float* w, float eps, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!hs || !y || !w || H <= 0) return CJ_ERR_ARG;
    cj::launch(norm_add_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, hs, y, w, eps, H);
    return launch_status();
}

CJ_EXPORT int cj_pair_embed(float* out, const void* table, const void* pair, int table_dtype, const int* ids,
                            const int* positions, const int* row_req, const int* req_start, const int* req_slot,
                            const int* state, int T, int H, int V, int buckets, long long mul_prev, long long mul_cur,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!out || !table || !pair || !ids || !positions || !row_req || !req_start || !req_slot || !state) return CJ_ERR_ARG;
    if (H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return CJ_ERR_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CJ_F32)
        cj::launch(pair_embed_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, (const float*)pair, ids,
                   positions, row_req, req_start, req_slot, state, H, V, buckets, mul_prev, mul_cur);
    else if (table_dtype == CJ_BF16)
        cj::launch(pair_embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table,
                   (const __nv_bfloat16*)pair, ids, positions, row_req, req_start, req_slot, state, H, V, buckets, mul_prev, mul_cur);
    else
        return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_pair_commit(const int* ids, const int* req_start, const int* req_slot, int* state, int requests,
                             cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (!ids || !req_start || !req_slot || !state) return CJ_ERR_ARG;
    cj::launch(pair_commit_kernel, dim3((requests + 63) / 64), dim3(64), 0, stream, ids, req_start, req_slot, state, requests);
    return launch_status();
}

CJ_EXPORT int cj_add_rows(float* hs, const float* other, const float* vec, int T, int H, cudaStream_t stream) {
    if (T <= 0 || (!other && !vec)) return 0;
    if (!hs || H <= 0) return CJ_ERR_ARG;
    cj::launch(add_rows_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, hs, other, vec, H);
    return launch_status();
}

CJ_EXPORT int cj_add_partials(float* hs, const float* parts, int n_parts, long long stride, long long n, cudaStream_t stream) {
    if (n <= 0 || n_parts <= 0) return 0;
    if (!hs || !parts) return CJ_ERR_ARG;
    const bool vec = (n | stride) % 4 == 0 && ((((uintptr_t)hs) | ((uintptr_t)parts)) & 15) == 0;
    long long blocks = (n / (vec ? 4 : 1) + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (vec) cj::launch(add_partials_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, stream, hs, parts, n_parts, stride, n);
    else cj::launch(add_partials_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, stream, hs, parts, n_parts, stride, n);
    return launch_status();
}

CJ_EXPORT int cj_gelu_gate(const float* a, int lda, const void* table, int table_dtype, int ldt, int offset, const int* ids, int V,
                           void* out, int out_dtype, int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    if (!a || !table || !ids || !out) return CJ_ERR_ARG;
    const int threads = n >= 256 ? 256 : (n >= 128 ? 128 : 64);
#define LAUNCH(TW, TO)                                                                                                       \
    cj::launch(gelu_gate_kernel<TW, TO>, dim3(T), dim3(threads), 0, stream, a, lda, (const TW*)table, ldt, offset, ids, V, \
               (TO*)out, n)
    if (table_dtype == CJ_F32 && out_dtype == CJ_F32) LAUNCH(float, float);
    else if (table_dtype == CJ_BF16 && out_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}
