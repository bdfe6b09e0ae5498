// The recurrence of a selective state-space mixer (state-space duality form, scalar decay per head),
// token by token in 32-bit, with the state of every sequence carried from step to step:
//
//   dt_t = softplus(raw_t + dt_bias_h)            a_h = exp(A_log_h)
//   S_t  = exp(-a_h dt_t) S_(t-1) + dt_t B_t x_t^T     (S: [N, P] per head)
//   y_t  = S_t^T C_t + D_h x_t,   then  y_t * silu(z_t)
//
// x [N_tok, heads, P], B and C [N_tok, groups, N] are columns of one 32-bit buffer (the filtered
// projection), z and the raw step sizes columns of another (the projection itself).  Head h reads group
// h / (heads / groups).  One block owns (sequence or chunk, head, 32 columns of S) and walks its tokens in order.
// Eight threads share two columns: a thread keeps N / 8 state elements of each in registers, so that a value of B
// or C read from shared memory serves both columns (the kernel is bound by those reads), and the eight add their
// parts of y by shuffles in a fixed order.  B and C of 16 tokens are staged in shared memory, each thread's part of
// N in a row of its own, padded so that the eight rows a warp reads in one 16-byte load fall into different
// banks.  A step of one token and a portion of a hundred run the same operations on the same numbers for every token.
//
// ssd_group_norm: the gated output in `parts` equal parts, each divided by its own root mean square,
// times a weight and a constant, stored in the storage type at a column offset of a wider buffer.
#include "common.cuh"

#define SSD_NS 8            // threads per column of the state (each holds two columns)
#define SSD_PB 32           // columns of the state per block
#define SSD_THREADS (SSD_NS * SSD_PB / 2)
#define SSD_CHUNK 16        // tokens staged in shared memory at a time
#define SSD_LCH 128         // tokens of a chunk when long portions are cut to run side by side

struct SsdArgs {
    const float* xbc; int xbc_stride; int x_col, b_col, c_col;    // filtered projection
    const float* proj; int proj_stride; int z_col, dt_col;        // projection: gate and raw step sizes
    const float* dt_bias; const float* a_log; const float* d_skip;
    float* state; long long state_stride;                          // state + slot * stride : [heads, N, P]
    float* y; int y_stride;                                        // [N_tok, heads * P] gated output
    const int* cu_q; const int* slots;
    int heads, groups, P, N;
    // long portions in chunks (see the kernel): the chunks' borders in packed tokens, each sequence's first chunk,
    // scratch for the chunks' states [n_chunks, heads, N, P] and the decays' running products [N_tok, heads]
    const int* chunk_t0; const int* seq_chunk0;
    float* chunk_state; float* cum;
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// MODE 0: a sequence's tokens of this step in order, from and to its state (single tokens, short portions).
// Long portions are cut into chunks of SSD_LCH tokens that run side by side:
// MODE 1: a chunk from a zero state: y_raw = (its own tokens' part of S)^T C + D x, not yet gated; the chunk's end
//         state to scratch; per token the product of the decays from the chunk's start (cum);
// (ssd_chunk_carry_kernel: chunk after chunk, S_in[c+1] = cum_end[c] S_in[c] + S_end[c], from and to the state)
// MODE 2: y = (y_raw + cum_t * S_in^T C_t) * silu(z): what the state before the chunk adds, then the gate.
// The sum over a token's past is the same sum, cut at the chunks' borders: equal up to rounding.
template <int NPT, int MODE, bool VEC>
__global__ void __launch_bounds__(SSD_THREADS) ssd_scan_kernel(SsdArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int h = blockIdx.y, p0 = blockIdx.z * SSD_PB;
    const int g = h / (a.heads / a.groups);
    // eight threads share two columns of S (pa, pb), each holding NPT of their N elements: a value of B or C that a
    // thread reads from shared memory serves both columns
    const int pl = threadIdx.x / SSD_NS, ns = threadIdx.x % SSD_NS;
    const int pa = p0 + pl, pb = pa + SSD_PB / 2;
    const bool live_a = pa < a.P, live_b = pb < a.P;
    int t0, t1;
    float* st;
    if (MODE == 0) {
        const int s = blockIdx.x;
        t0 = a.cu_q[s]; t1 = a.cu_q[s + 1];
        st = a.state + (size_t)a.slots[s] * a.state_stride + (size_t)h * a.N * a.P;
    } else {
        t0 = a.chunk_t0[blockIdx.x]; t1 = a.chunk_t0[blockIdx.x + 1];
        st = a.chunk_state + ((size_t)blockIdx.x * a.heads + h) * a.N * a.P;
    }
    constexpr int ROW = NPT + 4;                 // a thread's part of N, padded: the eight parts' rows fall into different banks
    constexpr int PADN = SSD_NS * NPT;           // N rounded up to what the eight threads hold
    float* sB = sm;                              // [CHUNK][8][ROW]   (MODE 2 stages C only)
    float* sC = sB + SSD_CHUNK * SSD_NS * ROW;   // [CHUNK][8][ROW]
    float* sX = sC + SSD_CHUNK * SSD_NS * ROW;   // [CHUNK][PB]
    float* sZ = sX + SSD_CHUNK * SSD_PB;         // [CHUNK][PB]
    float* sDt = sZ + SSD_CHUNK * SSD_PB;        // [CHUNK] step sizes, [CHUNK] decays
    float* sCum = sDt + 2 * SSD_CHUNK;           // [CHUNK] MODE 1: the decays' running product
    float* sY = sCum + SSD_CHUNK;                // [CHUNK][PB] a token's S^T C per column
    float2 Sa[NPT / 2], Sb[NPT / 2];             // state elements n = ns * NPT + 2 i, + 1 of columns pa and pb
#pragma unroll
    for (int i = 0; i < NPT / 2; ++i) {
        const int n = ns * NPT + 2 * i;
        const bool n0 = MODE != 1 && n < a.N, n1 = MODE != 1 && n + 1 < a.N;
        Sa[i].x = (n0 && live_a) ? st[(size_t)n * a.P + pa] : 0.f;
        Sa[i].y = (n1 && live_a) ? st[(size_t)(n + 1) * a.P + pa] : 0.f;
        Sb[i].x = (n0 && live_b) ? st[(size_t)n * a.P + pb] : 0.f;
        Sb[i].y = (n1 && live_b) ? st[(size_t)(n + 1) * a.P + pb] : 0.f;
    }
    const float neg_a = -expf(a.a_log[h]), dskip = a.d_skip[h], bias = a.dt_bias[h];
    float cum = 1.f;                             // MODE 1: product of the decays since the chunk's start
    for (int tc = t0; tc < t1; tc += SSD_CHUNK) {
        const int nt = min(SSD_CHUNK, t1 - tc);
        __syncthreads();
        // B and C of the chunk's tokens: eight loads of a thread in flight at a time
        if (VEC) {
            // 16-byte loads: i counts pieces of four state elements, PADN / 4 pieces per token (zeros past N)
            const int total = nt * (PADN / 4);
            for (int i0 = threadIdx.x; i0 < total; i0 += 8 * SSD_THREADS) {
                float4 vb[8], vc[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * SSD_THREADS;
                    const int tt = i / (PADN / 4), n = (i % (PADN / 4)) * 4;
                    const bool in = i < total && n < a.N;
                    const float* row = a.xbc + (size_t)(tc + tt) * a.xbc_stride + g * a.N + n;
                    vb[u] = vc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (MODE != 2 && in) vb[u] = *reinterpret_cast<const float4*>(row + a.b_col);
                    if (in) vc[u] = *reinterpret_cast<const float4*>(row + a.c_col);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * SSD_THREADS;
                    if (i < total) {
                        const int tt = i / (PADN / 4), n = (i % (PADN / 4)) * 4;
                        const int at = (tt * SSD_NS + n / NPT) * ROW + n % NPT;
                        if (MODE != 2) *reinterpret_cast<float4*>(sB + at) = vb[u];
                        *reinterpret_cast<float4*>(sC + at) = vc[u];
                    }
                }
            }
        } else {
            const int total = nt * PADN;
            for (int i0 = threadIdx.x; i0 < total; i0 += 8 * SSD_THREADS) {
                float vb[8], vc[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * SSD_THREADS;
                    const int tt = i / PADN, n = i % PADN;
                    const bool in = i < total && n < a.N;
                    const float* row = a.xbc + (size_t)(tc + tt) * a.xbc_stride + g * a.N + n;
                    vb[u] = (MODE != 2 && in) ? row[a.b_col] : 0.f;          // (zeros past N: those state elements stay zero)
                    vc[u] = in ? row[a.c_col] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * SSD_THREADS;
                    if (i < total) {
                        const int tt = i / PADN, n = i % PADN;
                        const int at = (tt * SSD_NS + n / NPT) * ROW + n % NPT;
                        if (MODE != 2) sB[at] = vb[u];
                        sC[at] = vc[u];
                    }
                }
            }
        }
        for (int i = threadIdx.x; i < nt * SSD_PB; i += blockDim.x) {
            const int tt = i / SSD_PB, pp = p0 + i % SSD_PB;
            const bool in = pp < a.P;
            if (MODE != 2) sX[i] = in ? a.xbc[(size_t)(tc + tt) * a.xbc_stride + a.x_col + h * a.P + pp] : 0.f;
            else sX[i] = in ? a.y[(size_t)(tc + tt) * a.y_stride + h * a.P + pp] : 0.f;          // y_raw
            if (MODE != 1) sZ[i] = in ? a.proj[(size_t)(tc + tt) * a.proj_stride + a.z_col + h * a.P + pp] : 0.f;
        }
        if (threadIdx.x < nt) {
            if (MODE == 2) {
                sDt[threadIdx.x] = a.cum[(size_t)(tc + threadIdx.x) * a.heads + h];
            } else {
                const float dt = softplus_f(a.proj[(size_t)(tc + threadIdx.x) * a.proj_stride + a.dt_col + h] + bias);
                sDt[threadIdx.x] = dt;
                sDt[SSD_CHUNK + threadIdx.x] = expf(neg_a * dt);
            }
        }
        __syncthreads();
        // the tokens in order: two state elements per instruction (fma.f32x2: each half rounds like a single fma),
        // a token's sum over a thread's part of N in four chains, (0 + 1) + (2 + 3), then over the eight threads
        for (int tt = 0; tt < nt; ++tt) {
            const float4* Ct = reinterpret_cast<const float4*>(sC + (tt * SSD_NS + ns) * ROW);
            float2 a01 = make_float2(0.f, 0.f), a23 = a01, b01 = a01, b23 = a01;
            if (MODE == 2) {
#pragma unroll
                for (int i = 0; i < NPT / 4; ++i) {
                    const float4 c = Ct[i];
                    const float2 c01 = make_float2(c.x, c.y), c23 = make_float2(c.z, c.w);
                    a01 = __ffma2_rn(Sa[2 * i], c01, a01); a23 = __ffma2_rn(Sa[2 * i + 1], c23, a23);
                    b01 = __ffma2_rn(Sb[2 * i], c01, b01); b23 = __ffma2_rn(Sb[2 * i + 1], c23, b23);
                }
            } else {
                const float decay = sDt[SSD_CHUNK + tt], dt = sDt[tt];
                const float dxa = dt * sX[tt * SSD_PB + pl], dxb = dt * sX[tt * SSD_PB + pl + SSD_PB / 2];
                const float2 decay2 = make_float2(decay, decay), dxa2 = make_float2(dxa, dxa), dxb2 = make_float2(dxb, dxb);
                const float4* Bt = reinterpret_cast<const float4*>(sB + (tt * SSD_NS + ns) * ROW);
#pragma unroll
                for (int i = 0; i < NPT / 4; ++i) {
                    const float4 b = Bt[i], c = Ct[i];
                    const float2 bq01 = make_float2(b.x, b.y), bq23 = make_float2(b.z, b.w);
                    const float2 c01 = make_float2(c.x, c.y), c23 = make_float2(c.z, c.w);
                    Sa[2 * i] = __ffma2_rn(decay2, Sa[2 * i], __fmul2_rn(dxa2, bq01));
                    Sa[2 * i + 1] = __ffma2_rn(decay2, Sa[2 * i + 1], __fmul2_rn(dxa2, bq23));
                    Sb[2 * i] = __ffma2_rn(decay2, Sb[2 * i], __fmul2_rn(dxb2, bq01));
                    Sb[2 * i + 1] = __ffma2_rn(decay2, Sb[2 * i + 1], __fmul2_rn(dxb2, bq23));
                    a01 = __ffma2_rn(Sa[2 * i], c01, a01); a23 = __ffma2_rn(Sa[2 * i + 1], c23, a23);
                    b01 = __ffma2_rn(Sb[2 * i], c01, b01); b23 = __ffma2_rn(Sb[2 * i + 1], c23, b23);
                }
                if (MODE == 1) {
                    cum *= decay;
                    if (threadIdx.x == 0) sCum[tt] = cum;
                }
            }
            float ya = (a01.x + a01.y) + (a23.x + a23.y), yb = (b01.x + b01.y) + (b23.x + b23.y);
#pragma unroll
            for (int o = 1; o < SSD_NS; o <<= 1) {
                ya += __shfl_xor_sync(0xffffffffu, ya, o);
                yb += __shfl_xor_sync(0xffffffffu, yb, o);
            }
            if (ns == 0) { sY[tt * SSD_PB + pl] = ya; sY[tt * SSD_PB + pl + SSD_PB / 2] = yb; }
        }
        __syncthreads();
        // what goes out for the chunk's tokens, every thread a few (token, column) pairs
        for (int i = threadIdx.x; i < nt * SSD_PB; i += blockDim.x) {
            const int tt = i / SSD_PB, pp = p0 + i % SSD_PB;
            if (pp >= a.P) continue;
            float yv;
            if (MODE == 2) yv = fmaf(sDt[tt], sY[i], sX[i]);          // y_raw + cum_t * (S_in^T C_t)
            else yv = fmaf(dskip, sX[i], sY[i]);
            if (MODE != 1) { const float z = sZ[i]; yv *= z / (1.0f + expf(-z)); }
            a.y[(size_t)(tc + tt) * a.y_stride + h * a.P + pp] = yv;
        }
        if (MODE == 1 && blockIdx.z == 0 && threadIdx.x < nt) a.cum[(size_t)(tc + threadIdx.x) * a.heads + h] = sCum[threadIdx.x];
    }
    if (MODE == 2) return;
#pragma unroll
    for (int i = 0; i < NPT / 2; ++i) {
        const int n = ns * NPT + 2 * i;
        if (live_a && n < a.N) st[(size_t)n * a.P + pa] = Sa[i].x;
        if (live_a && n + 1 < a.N) st[(size_t)(n + 1) * a.P + pa] = Sa[i].y;
        if (live_b && n < a.N) st[(size_t)n * a.P + pb] = Sb[i].x;
        if (live_b && n + 1 < a.N) st[(size_t)(n + 1) * a.P + pb] = Sb[i].y;
    }
}

// Between the two passes over the chunks: for every sequence, head and state element, chunk after chunk:
// what the chunk starts from takes the place of the chunk's own end state in scratch, and the state moves on:
// S <- cum_end[c] * S + S_end[c].  From the sequence's state, and back to it.
#define SSD_CARRY_BATCH 8
__global__ void __launch_bounds__(256) ssd_chunk_carry_kernel(SsdArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float cum_end[SSD_CARRY_BATCH];
    const int s = blockIdx.x, h = blockIdx.y;
    const int c0 = a.seq_chunk0[s], c1 = a.seq_chunk0[s + 1];
    const size_t per = (size_t)a.N * a.P;
    const size_t e = (size_t)blockIdx.z * blockDim.x + threadIdx.x;
    const bool live = e < per;
    float* st = a.state + (size_t)a.slots[s] * a.state_stride + (size_t)h * per + e;
    float S = live ? *st : 0.f;
    // a batch of chunks at a time: their loads are in flight together, only the sums are a chain
    for (int b0 = c0; b0 < c1; b0 += SSD_CARRY_BATCH) {
        const int nb = min(SSD_CARRY_BATCH, c1 - b0);
        __syncthreads();
        if (threadIdx.x < nb) cum_end[threadIdx.x] = a.cum[(size_t)(a.chunk_t0[b0 + threadIdx.x + 1] - 1) * a.heads + h];
        float end[SSD_CARRY_BATCH];
        float* cs = a.chunk_state + ((size_t)b0 * a.heads + h) * per + e;
#pragma unroll
        for (int u = 0; u < SSD_CARRY_BATCH; ++u) end[u] = (live && u < nb) ? cs[(size_t)u * a.heads * per] : 0.f;
        __syncthreads();
#pragma unroll
        for (int u = 0; u < SSD_CARRY_BATCH; ++u) {
            if (u < nb) {
                if (live) cs[(size_t)u * a.heads * per] = S;
                S = fmaf(cum_end[u], S, end[u]);
            }
        }
    }
    if (live) *st = S;
}

template <int MODE>
static int ssd_launch(const SsdArgs& a, dim3 grid, cudaStream_t stream) {
    const dim3 block(SSD_THREADS);
    const int npt = (a.N + SSD_NS - 1) / SSD_NS;
    const int npt_t = npt <= 4 ? 4 : npt <= 8 ? 8 : npt <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * SSD_CHUNK * SSD_NS * (npt_t + 4) + 3 * SSD_CHUNK * SSD_PB + 3 * SSD_CHUNK) * sizeof(float);
    // B and C in 16-byte loads where every row's pieces lie on 16-byte borders
    const bool vec = a.N % 4 == 0 && a.xbc_stride % 4 == 0 && a.b_col % 4 == 0 && a.c_col % 4 == 0 && ((uintptr_t)a.xbc & 15) == 0;
#define SSD_GO(NPT_) (vec ? idm_launch(ssd_scan_kernel<NPT_, MODE, true>, grid, block, smem, stream, a) \
                          : idm_launch(ssd_scan_kernel<NPT_, MODE, false>, grid, block, smem, stream, a))
    if (npt <= 4) SSD_GO(4);
    else if (npt <= 8) SSD_GO(8);
    else if (npt <= 16) SSD_GO(16);
    else SSD_GO(32);
#undef SSD_GO
    IDM_LAUNCH_CHECK("ssd_scan");
    return 0;
}

extern "C" int idm_ssd_chunk_tokens() { return SSD_LCH; }

// chunk_t0 [n_chunks + 1]: the chunks' first packed tokens (a chunk ends where the next begins; chunks never
// cross a sequence's border); seq_chunk0 [n_seqs + 1]: each sequence's first chunk; n_chunks == 0: every sequence
// token by token from its state.  scratch: n_chunks * heads * N * P floats, then n_tokens * heads.
extern "C" int idm_ssd_scan(const float* xbc, int xbc_stride, int x_col, int b_col, int c_col, const float* proj,
                            int proj_stride, int z_col, int dt_col, const float* dt_bias, const float* a_log,
                            const float* d_skip, float* state, long long state_stride, float* y, int y_stride,
                            const int* cu_q, const int* slots, int n_seqs, int heads, int groups, int P, int N,
                            const int* chunk_t0, const int* seq_chunk0, int n_chunks, float* scratch, int n_tokens,
                            cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    IDM_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && P > 0 && N > 0 && N <= 256,
                "ssd_scan: %d heads in %d groups, columns %d, state %d (at most 256)", heads, groups, P, N);
    IDM_REQUIRE(state_stride >= (long long)heads * N * P, "ssd_scan: a slot's state must hold %d x %d x %d floats", heads, N, P);
    IDM_REQUIRE(n_seqs <= 65535 && heads <= 65535, "ssd_scan: %d sequences, %d heads in one launch", n_seqs, heads);
    IDM_REQUIRE(n_chunks == 0 || (chunk_t0 && seq_chunk0 && scratch), "ssd_scan: chunks need their lists and scratch");
    SsdArgs a;
    a.xbc = xbc; a.xbc_stride = xbc_stride; a.x_col = x_col; a.b_col = b_col; a.c_col = c_col;
    a.proj = proj; a.proj_stride = proj_stride; a.z_col = z_col; a.dt_col = dt_col;
    a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip; a.state = state; a.state_stride = state_stride;
    a.y = y; a.y_stride = y_stride; a.cu_q = cu_q; a.slots = slots;
    a.heads = heads; a.groups = groups; a.P = P; a.N = N;
    a.chunk_t0 = chunk_t0; a.seq_chunk0 = seq_chunk0; a.chunk_state = scratch;
    a.cum = scratch ? scratch + (size_t)n_chunks * heads * N * P : nullptr;
    const int pz = (P + SSD_PB - 1) / SSD_PB;
    if (n_chunks == 0) return ssd_launch<0>(a, dim3(n_seqs, heads, pz), stream);
    if (ssd_launch<1>(a, dim3(n_chunks, heads, pz), stream)) return 1;
    idm_launch(ssd_chunk_carry_kernel, dim3(n_seqs, heads, (unsigned)(((size_t)N * P + 255) / 256)), dim3(256), 0, stream, a);
    IDM_LAUNCH_CHECK("ssd_chunk_carry");
    return ssd_launch<2>(a, dim3(n_chunks, heads, pz), stream);
}

// out[t, out_col + c] = y[t, c] / sqrt(mean over c's part of y^2 + eps) * w[c] * scale.  One warp per (token, part).
__global__ void __launch_bounds__(128) ssd_group_norm_kernel(const float* __restrict__ y, int width, int parts,
                                                             const float* __restrict__ w, float eps, float scale,
                                                             T* __restrict__ out, int out_stride, int out_col, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * parts) return;
    const int t = (int)(wid / parts), part = (int)(wid % parts), len = width / parts;
    const float* row = y + (size_t)t * width + (size_t)part * len;
    float ss = 0.f;
    for (int c = lane; c < len; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
    T* o = out + (size_t)t * out_stride + out_col + (size_t)part * len;
    const float* wp = w + (size_t)part * len;
    for (int c = lane; c < len; c += 32) from_f32(o[c], row[c] * inv * wp[c] * scale);
}

extern "C" int idm_ssd_group_norm(const float* y, int width, int parts, const float* w, float eps, float scale,
                                  void* out, int out_stride, int out_col, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && parts > 0 && width % parts == 0, "ssd_group_norm: %d columns in %d parts", width, parts);
    IDM_REQUIRE(out_col >= 0 && out_col + width <= out_stride, "ssd_group_norm: columns %d..%d of rows of %d", out_col,
                out_col + width, out_stride);
    const long long warps = (long long)n_tokens * parts;
    idm_launch(ssd_group_norm_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, y, width, parts, w, eps, scale,
               (T*)out, out_stride, out_col, n_tokens);
    IDM_LAUNCH_CHECK("ssd_group_norm");
    return 0;
}
