// Feed-forward experts chosen per token: out[t] = weight * sum_k down_e (act(gate_e x_t) * up_e x_t), e = the
// k-th expert of token t.  These kernels serve steps of few tokens (single tokens above all): every (token,
// choice) streams its expert's matrices once, a warp per output row, sums in 32-bit in a fixed order, so a
// token's result does not depend on what else the step holds.  Steps of many tokens group their rows by expert
// on the host and run one matrix product per expert instead; the kernels below then gather the rows
// (rows_gather) and add the experts' outputs back in the order of a token's choices (experts_combine).
#include "common.cuh"

// the experts of the step's tokens from a table by token id: choice[t, k] = table[tokens[t], k]
__global__ void __launch_bounds__(256) experts_from_table_kernel(const int* __restrict__ tokens, const int* __restrict__ table,
                                                                 int top, int* __restrict__ choice, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * top) choice[i] = table[(size_t)tokens[i / top] * top + i % top];
}

extern "C" int idm_experts_from_table(const int* tokens, const int* table, int top, int* choice, int n_tokens,
                                      cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(top > 0, "experts_from_table: top=%d", top);
    idm_launch(experts_from_table_kernel, dim3((n_tokens * top + 255) / 256), dim3(256), 0, stream, tokens, table, top, choice, n_tokens);
    IDM_LAUNCH_CHECK("experts_from_table");
    return 0;
}

__device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ xs, int K, int lane, bool vec) {
    float s = 0.f;
    if (vec) {
        constexpr int VN = Vec16<T>::N;
        for (int d = lane * VN; d < K; d += 32 * VN) {
            Vec16<T> wv; wv.load(w + d);
#pragma unroll
            for (int e = 0; e < VN; ++e) s = fmaf(xs[d + e], wv.get(e), s);
        }
    } else {
        for (int d = lane; d < K; d += 32) s = fmaf(xs[d], to_f32(w[d]), s);
    }
    return warp_sum(s);
}

// a[t, k, f] = act(gate_e[f] . x_t) * (up_e[f] . x_t), 32-bit; gate, up: [E, ff, width]; a block has one
// (token, choice) and 8 rows f per pass of its warps
__global__ void __launch_bounds__(256) experts_gate_up_kernel(const T* __restrict__ x, const int* __restrict__ choice,
                                                              const T* __restrict__ gate, const T* __restrict__ up,
                                                              float* __restrict__ a, int width, int ff, int top, int n_experts,
                                                              int act) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];
    const int tk = blockIdx.x;
    const int e = choice[tk];
    const int t = tk / top;
    for (int d = threadIdx.x; d < width; d += blockDim.x) xs[d] = to_f32(x[(size_t)t * width + d]);
    __syncthreads();
    if (e < 0 || e >= n_experts) return;                     // (a table entry outside the experts: contributes nothing)
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (width * (int)sizeof(T)) % 16 == 0;
    for (int f = blockIdx.y * 8 + wib; f < ff; f += gridDim.y * 8) {
        const size_t row = ((size_t)e * ff + f) * width;
        const float g = row_dot(gate + row, xs, width, lane, vec), u = row_dot(up + row, xs, width, lane, vec);
        if (lane == 0) a[(size_t)tk * ff + f] = gated_act(g, u, act);
    }
}

// h[t, w] += weight * sum_k down_e[w] . a[t, k];  down: [E, width, ff]; a block has one token, a warp an output row
__global__ void __launch_bounds__(256) experts_down_kernel(const float* __restrict__ a, const int* __restrict__ choice,
                                                           const T* __restrict__ down, float* __restrict__ h, int width,
                                                           int ff, int top, int n_experts, float weight) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float as[];                             // [top][ff]
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < top * ff; d += blockDim.x) as[d] = a[(size_t)t * top * ff + d];
    __syncthreads();
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (ff * (int)sizeof(T)) % 16 == 0;
    for (int w = blockIdx.y * 8 + wib; w < width; w += gridDim.y * 8) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = choice[t * top + k];
            if (e < 0 || e >= n_experts) continue;
            s += row_dot(down + ((size_t)e * width + w) * ff, as + k * ff, ff, lane, vec);
        }
        if (lane == 0) h[(size_t)t * width + w] += s * weight;
    }
}

extern "C" int idm_experts_few(const void* x, const int* choice, const void* gate, const void* up, const void* down,
                               float* a, float* h, int n_tokens, int width, int ff, int top, int n_experts, int act,
                               float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && ff > 0 && top > 0 && n_experts > 0 && (act == 0 || act == 1), "experts: width=%d ff=%d top=%d experts=%d act=%d",
                width, ff, top, n_experts, act);
    IDM_REQUIRE((size_t)width * 4 <= 160 * 1024 && (size_t)top * ff * 4 <= 160 * 1024, "experts: width=%d or top * ff=%d does not fit shared memory",
                width, top * ff);
    const size_t s1 = (size_t)width * 4, s2 = (size_t)top * ff * 4;
    if (s1 > 48 * 1024) cudaFuncSetAttribute(experts_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    if (s2 > 48 * 1024) cudaFuncSetAttribute(experts_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2);
    // blocks along the rows: enough to fill the part for one token, fewer per token as tokens grow
    const int by1 = max(1, min((ff + 7) / 8, 592 / max(1, n_tokens * top)));
    const int by2 = max(1, min((width + 7) / 8, 592 / max(1, n_tokens)));
    idm_launch(experts_gate_up_kernel, dim3(n_tokens * top, by1), dim3(256), s1, stream, (const T*)x, choice, (const T*)gate,
               (const T*)up, a, width, ff, top, n_experts, act);
    IDM_LAUNCH_CHECK("experts_gate_up");
    idm_launch(experts_down_kernel, dim3(n_tokens, by2), dim3(256), s2, stream, (const float*)a, choice, (const T*)down, h, width,
               ff, top, n_experts, weight);
    IDM_LAUNCH_CHECK("experts_down");
    return 0;
}

// out[i, :] = x[src[i], :]  (rows of the storage type; a step's rows in the order of their experts)
__global__ void __launch_bounds__(256) rows_gather_kernel(const T* __restrict__ x, const int* __restrict__ src, T* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = blockIdx.x;
    const T* r = x + (size_t)src[i] * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) out[i * width + d] = r[d];
}

extern "C" int idm_rows_gather(const void* x, const int* src, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    idm_launch(rows_gather_kernel, dim3(n_rows), dim3(256), 0, stream, (const T*)x, src, (T*)out, width);
    IDM_LAUNCH_CHECK("rows_gather");
    return 0;
}

// h[t, :] += weight * sum_k z[place[t, k], :] in ascending k  (z 32-bit: the experts' outputs, grouped rows)
__global__ void __launch_bounds__(256) experts_combine_kernel(const float* __restrict__ z, const int* __restrict__ place,
                                                              float* __restrict__ h, int width, int top, float weight) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int r = place[t * top + k];
            if (r >= 0) s += z[(size_t)r * width + d];
        }
        h[t * width + d] += s * weight;
    }
}

extern "C" int idm_experts_combine(const float* z, const int* place, float* h, int n_tokens, int width, int top,
                                   float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    idm_launch(experts_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, z, place, h, width, top, weight);
    IDM_LAUNCH_CHECK("experts_combine");
    return 0;
}
