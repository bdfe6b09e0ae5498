// Attention through a latent: what a token keeps is ONE row [c | r] for all heads, c a normed vector of `R`
// numbers from which every head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), r a rotated key
// part of `dr` numbers that all heads share.  With a head's query split as [qn | qr], its score against token j is
//
//     s = (qn . Uk_h c_j + qr . r_j) * scale = ((Uk_h^T qn) . c_j + qr . r_j) * scale
//
// so a step's queries are first carried into the latent's space (`headwise_kernel`: qa = [Uk_h^T qn | turn(qr)]),
// every head then reads the same cached rows (`latent_attention_kernel`: scores against [c | r], the context
// as a weighted sum of c), and the head's value map is applied once to the context (`headwise_kernel`).  The
// cache is read once per token and step whatever the number of heads.  All arithmetic here is 32-bit; the cache
// rows and the value maps' outputs are in the storage type.
//
// Rotation: neighbours (2i, 2i+1) of the rotated part are turned by the token's angle i, (u, v) ->
// (u cos - v sin, v cos + u sin), cos and sin from the step's table times a constant magnitude.
#include "common.cuh"

// ------------------------------------------------------------------ the row a token keeps
// proj [N, ld] 32-bit, columns col0 .. col0 + R: the latent before its norm; the next dr: the shared key part.
// One block per token: c = x / sqrt(mean(x^2) + eps) * w, r turned; [c | r] to the token's place in the paged
// pool [pages, PAGE, R + dr] and, if asked for, to packed rows row_out [N, R + dr] (the step's own keys).
__global__ void __launch_bounds__(128) latent_kv_finish_kernel(const float* __restrict__ proj, int ld, int col0, int R, int dr,
                                                               int rot_dims, const float* __restrict__ w, float eps,
                                                               const float2* __restrict__ cs, int half, float mag,
                                                               T* __restrict__ pool, const int* __restrict__ table,
                                                               int table_stride, const int* __restrict__ token_seq,
                                                               const int* __restrict__ positions, const int* __restrict__ slots,
                                                               T* __restrict__ row_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* x = proj + (size_t)t * ld + col0;
    float ss = 0.f;
    for (int d = threadIdx.x; d < R; d += blockDim.x) ss = fmaf(x[d], x[d], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
    const int pos = positions[t], slot = slots[token_seq[t]];
    const int page = table[(size_t)slot * table_stride + pos / IDM_PAGE];
    T* row = pool + ((size_t)page * IDM_PAGE + pos % IDM_PAGE) * (size_t)(R + dr);
    T* row2 = row_out ? row_out + (size_t)t * (R + dr) : nullptr;
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        const float c = x[d] * inv * w[d];
        from_f32(row[d], c);
        if (row2) from_f32(row2[d], c);
    }
    const float* xr = x + R;
    for (int i = threadIdx.x; 2 * i < dr; i += blockDim.x) {
        float u = xr[2 * i], v = (2 * i + 1 < dr) ? xr[2 * i + 1] : 0.f;
        if (2 * i + 1 < rot_dims) {
            const float2 a = cs[(size_t)t * half + i];
            const float co = a.x * mag, si = a.y * mag;
            const float u2 = u * co - v * si, v2 = v * co + u * si;
            u = u2; v = v2;
        }
        from_f32(row[R + 2 * i], u);
        if (row2) from_f32(row2[R + 2 * i], u);
        if (2 * i + 1 < dr) {
            from_f32(row[R + 2 * i + 1], v);
            if (row2) from_f32(row2[R + 2 * i + 1], v);
        }
    }
}

extern "C" int idm_latent_kv_finish(const float* proj, int ld, int col0, int R, int dr, int rot_dims, const float* w,
                                    float eps, const float* cs, int half, float mag, void* pool, const int* table,
                                    int table_stride, const int* token_seq, const int* positions, const int* slots,
                                    void* row_out, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(R > 0 && dr >= 0 && col0 >= 0 && col0 + R + dr <= ld, "latent_kv_finish: columns %d + %d + %d of %d", col0, R, dr, ld);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "latent_kv_finish: %d turned dims of %d with a table of %d angles", rot_dims, dr, half);
    idm_launch(latent_kv_finish_kernel, dim3(n_tokens), dim3(128), 0, stream, proj, ld, col0, R, dr, rot_dims, w, eps,
               (const float2*)cs, half, mag, (T*)pool, table, table_stride, token_seq, positions, slots, (T*)row_out);
    IDM_LAUNCH_CHECK("latent_kv_finish");
    return 0;
}

// ------------------------------------------------------------------ a matrix per head
// out[t, h, o] = sum_i x[t, h, i] * W[h, i, o] for every head h on its own: x 32-bit with strides of its own, W
// [H, I, O] in the storage type (o contiguous).  A block has one head, 32 outputs and up to HW_TOKENS tokens; its
// eight warps each take an eighth of the i (a lane owns an output and reads W side by side with its neighbours),
// and the eight partial sums of an element are added in ascending order, so the order of every sum depends on I
// alone.  `tail` more columns of x behind the I are copied behind the O outputs, the first `rot_dims` of them
// turned by the token's angles (a query's rotated part).  A head's matrix is read once per HW_TOKENS tokens.
#define HW_TOKENS 8
#define HW_WARPS 8          // (warp w also adds token w's partial sums: as many warps as tokens)
static_assert(HW_WARPS == HW_TOKENS, "a warp per token in the last phase");

template <typename OutT>
__global__ void __launch_bounds__(HW_WARPS * 32) headwise_kernel(const float* __restrict__ x, long long x_tok, int x_head, int I,
                                                                 const T* __restrict__ W, int O, OutT* __restrict__ out,
                                                                 long long o_tok, int o_head, int tail, int rot_dims,
                                                                 const float2* __restrict__ cs, int half, float mag, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];                       // [HW_TOKENS][I], then the warps' partial sums [HW_WARPS][HW_TOKENS][32]
    float* part = xs + HW_TOKENS * I;
    const int h = blockIdx.y, t0 = blockIdx.x * HW_TOKENS, o0 = blockIdx.z * 32;
    const int nt = min(HW_TOKENS, n_tokens - t0);
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < HW_TOKENS * I; e += blockDim.x) {
        const int tt = e / I, i = e % I;
        xs[e] = tt < nt ? x[(size_t)(t0 + tt) * x_tok + (size_t)h * x_head + i] : 0.f;
    }
    __syncthreads();
    const int o = o0 + lane;
    const int per = (I + HW_WARPS - 1) / HW_WARPS, i0 = wib * per, i1 = min(I, i0 + per);
    float acc[HW_TOKENS];
#pragma unroll
    for (int tt = 0; tt < HW_TOKENS; ++tt) acc[tt] = 0.f;
    if (o < O) {
        const T* Wh = W + (size_t)h * I * O + o;
#pragma unroll 8
        for (int i = i0; i < i1; ++i) {
            const float wv = to_f32(Wh[(size_t)i * O]);
#pragma unroll
            for (int tt = 0; tt < HW_TOKENS; ++tt) acc[tt] = fmaf(xs[tt * I + i], wv, acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < HW_TOKENS; ++tt) part[(wib * HW_TOKENS + tt) * 32 + lane] = acc[tt];
    __syncthreads();
    {   // warp w adds token w's eight partial sums, in the order of the warps that made them
        const int tt = wib;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < HW_WARPS; ++w) s += part[(w * HW_TOKENS + tt) * 32 + lane];
        if (tt < nt && o < O) from_f32(out[(size_t)(t0 + tt) * o_tok + (size_t)h * o_head + o], s);
    }
    if (blockIdx.z != 0) return;
    for (int e = threadIdx.x; e < nt * ((tail + 1) / 2); e += blockDim.x) {
        const int tt = e / ((tail + 1) / 2), i = e % ((tail + 1) / 2), t = t0 + tt;
        const float* xr = x + (size_t)t * x_tok + (size_t)h * x_head + I;
        OutT* orow = out + (size_t)t * o_tok + (size_t)h * o_head + O;
        float u = xr[2 * i], v = (2 * i + 1 < tail) ? xr[2 * i + 1] : 0.f;
        if (2 * i + 1 < rot_dims) {
            const float2 a = cs[(size_t)t * half + i];
            const float co = a.x * mag, si = a.y * mag;
            const float u2 = u * co - v * si, v2 = v * co + u * si;
            u = u2; v = v2;
        }
        from_f32(orow[2 * i], u);
        if (2 * i + 1 < tail) from_f32(orow[2 * i + 1], v);
    }
}

// out_is_f32: the outputs are 32-bit (queries in the latent's space); else the storage type (a product's input)
extern "C" int idm_headwise(const float* x, long long x_tok, int x_head, int I, const void* W, int O, void* out,
                            int out_is_f32, long long o_tok, int o_head, int tail, int rot_dims, const float* cs, int half,
                            float mag, int n_tokens, int n_heads, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(I > 0 && O >= 0 && n_heads > 0 && tail >= 0, "headwise: sizes I=%d O=%d heads=%d tail=%d", I, O, n_heads, tail);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= tail && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "headwise: %d turned dims of %d with a table of %d angles", rot_dims, tail, half);
    const size_t smem = ((size_t)HW_TOKENS * I + HW_WARPS * HW_TOKENS * 32) * sizeof(float);
    IDM_REQUIRE(smem <= 200 * 1024, "headwise: I=%d does not fit shared memory", I);
    const dim3 grid((n_tokens + HW_TOKENS - 1) / HW_TOKENS, n_heads, max(1, (O + 31) / 32));
    IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "headwise: %d heads, %d outputs", n_heads, O);
    if (out_is_f32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(headwise_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        idm_launch(headwise_kernel<float>, grid, dim3(HW_WARPS * 32), smem, stream, x, x_tok, x_head, I, (const T*)W, O, (float*)out,
                   o_tok, o_head, tail, rot_dims, (const float2*)cs, half, mag, n_tokens);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(headwise_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        idm_launch(headwise_kernel<T>, grid, dim3(HW_WARPS * 32), smem, stream, x, x_tok, x_head, I, (const T*)W, O, (T*)out,
                   o_tok, o_head, tail, rot_dims, (const float2*)cs, half, mag, n_tokens);
    }
    IDM_LAUNCH_CHECK("headwise");
    return 0;
}

// ------------------------------------------------------------------ attention over the latent rows
// A block has one query token, up to LA_WARPS warps of one head each (two each when the layer has more than
// LA_WARPS heads) and one run of keys: positions
// [run * run_keys, (run + 1) * run_keys) up to the query's own.  Keys are walked in blocks of 32 at absolute
// positions, staged in shared memory once for all the block's heads (two buffers: the next block's copies run
// while this one is scored); lane i scores key j0 + i against the head's
// query (kept in shared memory, 32-bit), the running (max, sum, context) is rescaled block by block, and the
// context is a weighted sum of the rows' first R numbers, a lane owning pairs of neighbours.  With one run the
// block finishes the row (the sink, a score with no key and no value, joins the sum once) and writes the context
// [N, H, R] in 32-bit; with several, every run leaves (max, sum, context) in scratch and latent_fold_kernel adds
// the runs in ascending order.
#define LA_WARPS 8

struct LatentArgs {
    const float* qa;          // [N, H, D]
    const T* pool;            // [pages, PAGE, D]
    const int* table; int table_stride;
    const int* token_seq; const int* positions; const int* slots;
    const float* sink;        // [H] or null
    float* ctx;               // [N, H, R]
    float* part;              // [N, H, n_runs, R + 2]: (max, sum, context) of each run
    int n_tokens, H, R, D;
    float scale;
    int run_keys, n_runs, stride_words, n_buf;
};

template <int NACC, int HPW>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(LatentArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);                          // [LA_WARPS * HPW][D] (rows padded to 4 floats)
    const int Dq = (a.D + 3) & ~3;
    uint32_t* tile = reinterpret_cast<uint32_t*>(qs + LA_WARPS * HPW * Dq);  // [buffers][32][stride_words]
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a warp has HPW heads side by side: a key's row is read once from shared memory for all of them
    const int t = blockIdx.x, head = (blockIdx.y * LA_WARPS + wib) * HPW, run = blockIdx.z;
    const bool live_head = head < a.H;
    const int nh = min(HPW, a.H - head);                                      // (heads of this warp that exist)
    const int pos = a.positions[t], slot = a.slots[a.token_seq[t]];
    const int lo = run * a.run_keys, hi = min(pos, lo + a.run_keys - 1);      // keys lo .. hi
    float m[HPW], l[HPW];
    float acc[HPW][NACC];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[hh][i] = 0.f;
    }
    if (lo <= pos) {
        if (live_head) {
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) {
                const float* q = a.qa + ((size_t)t * a.H + min(head + hh, a.H - 1)) * a.D;
                for (int d = lane; d < Dq; d += 32) qs[(wib * HPW + hh) * Dq + d] = d < a.D ? q[d] : 0.f;
            }
        }
        const int row_bytes = a.D * (int)sizeof(T);
        const bool vec = (row_bytes % 16) == 0;
        const int* pages = a.table + (size_t)slot * a.table_stride;
        const int n_tiles = (hi - lo) / 32 + 1;
        // a block of 32 keys into one of the staging buffers: 16-byte pieces by asynchronous copies (the next
        // block's are in flight while this one is scored), rows off the 16-byte borders element by element
        auto stage = [&](int buf, int it) {
            const int j0 = lo + it * 32, nk = min(32, hi - j0 + 1);
            uint32_t* dst = tile + (size_t)buf * 32 * a.stride_words;
            if (vec) {
                const int cpr = row_bytes / 16;
                for (int c = threadIdx.x; c < nk * cpr; c += LA_WARPS * 32) {
                    const int r = c / cpr, cc = c % cpr, j = j0 + r;
                    const T* src = a.pool + ((size_t)pages[j / IDM_PAGE] * IDM_PAGE + j % IDM_PAGE) * (size_t)a.D;
                    const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst + (size_t)r * a.stride_words + cc * 4);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(reinterpret_cast<const uint4*>(src) + cc) : "memory");
                }
            } else {
                T* tl = reinterpret_cast<T*>(dst);
                const int stride_e = a.stride_words * 4 / (int)sizeof(T);
                for (int c = threadIdx.x; c < nk * a.D; c += LA_WARPS * 32) {
                    const int r = c / a.D, d = c % a.D, j = j0 + r;
                    tl[(size_t)r * stride_e + d] = a.pool[((size_t)pages[j / IDM_PAGE] * IDM_PAGE + j % IDM_PAGE) * (size_t)a.D + d];
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (a.n_buf == 2) stage(0, 0);
        for (int it = 0; it < n_tiles; ++it) {
            const int j0 = lo + it * 32, nk = min(32, hi - j0 + 1);
            int buf = 0;
            if (a.n_buf == 2) {
                buf = it & 1;
                if (it + 1 < n_tiles) {
                    stage(buf ^ 1, it + 1);
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                } else {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                }
            } else {
                stage(0, it);
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();                                                  // the block of keys (and, at first, qs) is there
            const uint32_t* cur = tile + (size_t)buf * 32 * a.stride_words;
            if (live_head) {
                const bool valid = lane < nk;
                float sc[HPW], p[HPW];
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) sc[hh] = -INFINITY;
                if (valid) {
                    const T* krow = reinterpret_cast<const T*>(cur + (size_t)lane * a.stride_words);
                    const float* q = qs + wib * HPW * Dq;
                    float d0[HPW], d1[HPW];
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) d0[hh] = d1[hh] = 0.f;
                    constexpr int VN = Vec16<T>::N;
                    int d = 0;
                    for (; d + VN <= a.D; d += VN) {
                        Vec16<T> kv; kv.load(krow + d);
#pragma unroll
                        for (int hh = 0; hh < HPW; ++hh) {
#pragma unroll
                            for (int e = 0; e < VN; e += 4) {                 // (a query's row starts on a 16-byte border)
                                const float4 q4 = *reinterpret_cast<const float4*>(q + hh * Dq + d + e);
                                d0[hh] = fmaf(q4.x, kv.get(e), d0[hh]);
                                d1[hh] = fmaf(q4.y, kv.get(e + 1), d1[hh]);
                                d0[hh] = fmaf(q4.z, kv.get(e + 2), d0[hh]);
                                d1[hh] = fmaf(q4.w, kv.get(e + 3), d1[hh]);
                            }
                        }
                    }
                    for (; d < a.D; ++d)
#pragma unroll
                        for (int hh = 0; hh < HPW; ++hh) d0[hh] = fmaf(q[hh * Dq + d], to_f32(krow[d]), d0[hh]);
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) sc[hh] = (d0[hh] + d1[hh]) * a.scale;
                }
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) {
                    const float m_new = fmaxf(m[hh], warp_max(sc[hh]));
                    const float alpha = expf(m[hh] - m_new);                  // (m = -inf at first: 0)
                    p[hh] = valid ? expf(sc[hh] - m_new) : 0.f;
                    l[hh] = l[hh] * alpha + warp_sum(p[hh]);
                    m[hh] = m_new;
#pragma unroll
                    for (int i = 0; i < NACC; ++i) acc[hh][i] *= alpha;
                }
                for (int jj = 0; jj < nk; ++jj) {
                    float pj[HPW];
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) pj[hh] = __shfl_sync(0xffffffffu, p[hh], jj);
                    const T* crow = reinterpret_cast<const T*>(cur + (size_t)jj * a.stride_words);
#pragma unroll
                    for (int i = 0; i < NACC / 2; ++i) {
                        const int d = 2 * lane + 64 * i;
                        if (d < a.R) {                                        // (d + 1 may be R: inside the row, never stored)
                            float c0, c1;
                            if (sizeof(T) == 2) {
                                const uint32_t wv = *reinterpret_cast<const uint32_t*>(crow + d);
                                c0 = __uint_as_float(wv << 16); c1 = __uint_as_float(wv & 0xffff0000u);
                            } else {
                                const float2 cv = *reinterpret_cast<const float2*>(crow + d);
                                c0 = cv.x; c1 = cv.y;
                            }
#pragma unroll
                            for (int hh = 0; hh < HPW; ++hh) {
                                acc[hh][2 * i] = fmaf(pj[hh], c0, acc[hh][2 * i]);
                                acc[hh][2 * i + 1] = fmaf(pj[hh], c1, acc[hh][2 * i + 1]);
                            }
                        }
                    }
                }
            }
            __syncthreads();                                                  // everyone is done with this buffer
        }
    }
    if (!live_head) return;
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        if (hh >= nh) break;
        const int hd = head + hh;
        if (a.n_runs == 1) {
            const float sk = a.sink ? a.sink[hd] : -INFINITY;
            const float mf = fmaxf(m[hh], sk);
            const float w = expf(m[hh] - mf);
            const float inv = 1.0f / (l[hh] * w + (a.sink ? expf(sk - mf) : 0.f));
            float* o = a.ctx + ((size_t)t * a.H + hd) * a.R;
#pragma unroll
            for (int i = 0; i < NACC / 2; ++i) {
                const int d = 2 * lane + 64 * i;
                if (d < a.R) o[d] = acc[hh][2 * i] * w * inv;
                if (d + 1 < a.R) o[d + 1] = acc[hh][2 * i + 1] * w * inv;
            }
        } else {
            float* o = a.part + (((size_t)t * a.H + hd) * a.n_runs + run) * (size_t)(a.R + 2);
            if (lane == 0) { o[0] = m[hh]; o[1] = l[hh]; }
            if (lo <= pos) {
#pragma unroll
                for (int i = 0; i < NACC / 2; ++i) {
                    const int d = 2 * lane + 64 * i;
                    if (d < a.R) o[2 + d] = acc[hh][2 * i];
                    if (d + 1 < a.R) o[2 + d + 1] = acc[hh][2 * i + 1];
                }
            }
        }
    }
}

#if defined(IDM_BF16)
// ------------------------------------------------------------------ the same on tensor-core fragments (bfloat16)
// For latents whose rows are whole 16-element steps (D % 16 == 0, R % 32 == 0, R <= 512).  A block of four warps has one
// query token, sixteen heads (the rows of an m16n8k16 tile; rows of heads that do not exist are zero) and one run of
// keys.  Per block of 32 keys: warp w scores keys 8w .. 8w+7 for all sixteen heads (queries and keys as bfloat16
// fragments from shared memory, 32-bit sums), the rows' maxima and sums meet across the warps in shared memory,
// the weights go to shared memory as bfloat16, and warp w adds the weighted rows' columns [w R/4, (w+1) R/4) to
// its part of the context.  Runs, scratch and the sink are those of the kernel above.
#define LM_WARPS 4

__device__ __forceinline__ void lm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <int NT_MAX>
__global__ void __launch_bounds__(LM_WARPS * 32) latent_attention_mma_kernel(LatentArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DS = a.stride_words * 2;                                        // row stride of the staged rows in elements (16 bytes x an odd number)
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [16][DS]
    __nv_bfloat16* Ks = Qs + 16 * DS;                                         // [2][32][DS]
    __nv_bfloat16* Ps = Ks + 2 * 32 * DS;                                     // [16][40]
    float* red_max = reinterpret_cast<float*>(Ps + 16 * 40);                  // [LM_WARPS][16]
    float* red_sum = red_max + LM_WARPS * 16;                                 // [LM_WARPS][16]
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c2 = (lane & 3) * 2;
    const int t = blockIdx.x, head0 = blockIdx.y * 16, run = blockIdx.z;
    const int nh = min(16, a.H - head0);
    const int pos = a.positions[t], slot = a.slots[a.token_seq[t]];
    const int lo = run * a.run_keys, hi = min(pos, lo + a.run_keys - 1);
    const int NT = a.R / 32;                                                  // 8-column tiles of the context a warp owns
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};                   // rows g and g + 8
    float o[NT_MAX][4];
#pragma unroll
    for (int nt = 0; nt < NT_MAX; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    if (lo <= pos) {
        for (int e = threadIdx.x; e < 16 * a.D; e += LM_WARPS * 32) {
            const int r = e / a.D, d = e % a.D;
            Qs[r * DS + d] = __float2bfloat16_rn(r < nh ? a.qa[((size_t)t * a.H + head0 + r) * a.D + d] : 0.f);
        }
        const int* pages = a.table + (size_t)slot * a.table_stride;
        const int n_tiles = (hi - lo) / 32 + 1, cpr = a.D / 8;
        auto stage = [&](int buf, int it) {
            const int j0 = lo + it * 32, nk = min(32, hi - j0 + 1);
            __nv_bfloat16* dst = Ks + (size_t)buf * 32 * DS;
            for (int c = threadIdx.x; c < 32 * cpr; c += LM_WARPS * 32) {
                const int r = c / cpr, cc = c % cpr;
                if (r < nk) {
                    const int j = j0 + r;
                    const T* src = a.pool + ((size_t)pages[j / IDM_PAGE] * IDM_PAGE + j % IDM_PAGE) * (size_t)a.D;
                    const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst + (size_t)r * DS + cc * 8);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(reinterpret_cast<const uint4*>(src) + cc) : "memory");
                } else {                                                      // rows behind the last key: zeros (their weights are 0, and 0 x anything finite is 0)
                    *reinterpret_cast<uint4*>(dst + (size_t)r * DS + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        stage(0, 0);
        const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (lane & 15) * DS + (lane >> 4) * 8);
        const uint32_t p_addr = (uint32_t)__cvta_generic_to_shared(Ps + (lane & 15) * 40 + (lane >> 4) * 8);
        for (int it = 0; it < n_tiles; ++it) {
            const int j0 = lo + it * 32, buf = it & 1;
            if (it + 1 < n_tiles) {
                stage(buf ^ 1, it + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();                                                  // (a) the keys (and, at first, the queries) are there
            const __nv_bfloat16* Kb = Ks + (size_t)buf * 32 * DS;
            // scores of keys 8w .. 8w+7: two 16-element steps of the rows per fragment load
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Kb + (8 * w + (lane & 7)) * DS);
            const int steps = a.D / 16;
            for (int kk = 0; kk < steps; kk += 2) {
                uint32_t qa0[4], qa1[4], kb[4];
                const bool two = kk + 1 < steps;
                lm_ldmatrix_x4(kb, k_addr + (kk * 16 + (two ? (lane >> 3) * 8 : ((lane >> 3) & 1) * 8)) * 2);
                lm_ldmatrix_x4(qa0, q_addr + kk * 32);
                lm_mma(sc, qa0, kb[0], kb[1]);
                if (two) {
                    lm_ldmatrix_x4(qa1, q_addr + (kk + 1) * 32);
                    lm_mma(sc, qa1, kb[2], kb[3]);
                }
            }
            const int j = j0 + 8 * w + c2;                                     // this lane's keys: j, j + 1 (rows g and g + 8)
            const bool v0 = j <= hi, v1 = j + 1 <= hi;
            sc[0] = v0 ? sc[0] * a.scale : -INFINITY; sc[1] = v1 ? sc[1] * a.scale : -INFINITY;
            sc[2] = v0 ? sc[2] * a.scale : -INFINITY; sc[3] = v1 ? sc[3] * a.scale : -INFINITY;
            float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]);
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            if ((lane & 3) == 0) { red_max[w * 16 + g] = mx0; red_max[w * 16 + g + 8] = mx1; }
            __syncthreads();                                                  // (b)
            float mn0 = m[0], mn1 = m[1];
#pragma unroll
            for (int ww = 0; ww < LM_WARPS; ++ww) { mn0 = fmaxf(mn0, red_max[ww * 16 + g]); mn1 = fmaxf(mn1, red_max[ww * 16 + g + 8]); }
            const float al0 = expf(m[0] - mn0), al1 = expf(m[1] - mn1);        // (the first block of a run holds a key: the maxima are finite)
            const float p0 = v0 ? expf(sc[0] - mn0) : 0.f, p1 = v1 ? expf(sc[1] - mn0) : 0.f;
            const float p2 = v0 ? expf(sc[2] - mn1) : 0.f, p3 = v1 ? expf(sc[3] - mn1) : 0.f;
            float s0 = p0 + p1, s1 = p2 + p3;
            s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
            s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
            if ((lane & 3) == 0) { red_sum[w * 16 + g] = s0; red_sum[w * 16 + g + 8] = s1; }
            *reinterpret_cast<__nv_bfloat162*>(Ps + g * 40 + 8 * w + c2) = __floats2bfloat162_rn(p0, p1);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * 40 + 8 * w + c2) = __floats2bfloat162_rn(p2, p3);
            __syncthreads();                                                  // (c) weights and sums are there
            float t0 = 0.f, t1 = 0.f;
#pragma unroll
            for (int ww = 0; ww < LM_WARPS; ++ww) { t0 += red_sum[ww * 16 + g]; t1 += red_sum[ww * 16 + g + 8]; }
            l[0] = l[0] * al0 + t0; l[1] = l[1] * al1 + t1;
            m[0] = mn0; m[1] = mn1;
            uint32_t pa0[4], pa1[4];
            lm_ldmatrix_x4(pa0, p_addr);                                      // keys 0 .. 15 of the block
            lm_ldmatrix_x4(pa1, p_addr + 32);                                 // keys 16 .. 31
            const uint32_t c_addr = (uint32_t)__cvta_generic_to_shared(Kb + lane * DS + w * (a.R / 4));
#pragma unroll
            for (int nt = 0; nt < NT_MAX; ++nt) {
                if (nt < NT) {
                    o[nt][0] *= al0; o[nt][1] *= al0; o[nt][2] *= al1; o[nt][3] *= al1;
                    uint32_t cb[4];
                    lm_ldmatrix_x4_trans(cb, c_addr + nt * 16);               // lane = key: rows 0..31 of 8 columns
                    lm_mma(o[nt], pa0, cb[0], cb[1]);
                    lm_mma(o[nt], pa1, cb[2], cb[3]);
                }
            }
            __syncthreads();                                                  // (d) everyone is done with this buffer, the weights and the sums
        }
    }
    // rows g and g + 8 of this lane: heads head0 + g, head0 + g + 8; its columns: w R/4 + nt * 8 + c2, + 1
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
        if (r >= nh) continue;
        const int hd = head0 + r;
        if (a.n_runs == 1) {
            const float sk = a.sink ? a.sink[hd] : -INFINITY;
            const float mf = fmaxf(m[half], sk);
            const float wgt = expf(m[half] - mf);
            const float inv = wgt / (l[half] * wgt + (a.sink ? expf(sk - mf) : 0.f));
            float* out = a.ctx + ((size_t)t * a.H + hd) * a.R + w * (a.R / 4) + c2;
#pragma unroll
            for (int nt = 0; nt < NT_MAX; ++nt)
                if (nt < NT) *reinterpret_cast<float2*>(out + nt * 8) = make_float2(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
        } else {
            float* out = a.part + (((size_t)t * a.H + hd) * a.n_runs + run) * (size_t)(a.R + 2);
            if (w == 0 && (lane & 3) == 0) { out[0] = m[half]; out[1] = l[half]; }
            if (lo <= pos) {
#pragma unroll
                for (int nt = 0; nt < NT_MAX; ++nt)
                    if (nt < NT) *reinterpret_cast<float2*>(out + 2 + w * (a.R / 4) + nt * 8 + c2) = make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
            }
        }
    }
}
#endif

// one block per (token, head): the runs' maxima and sums are gathered by the first warp, a run per lane, every run's
// weight is computed once and kept in shared memory, and a thread adds its columns of the runs' contexts in ascending
// order of the runs (eight loads in flight); the sink joins the sum once
#define LF_MAX_RUNS 512
#define LF_THREADS 256
__global__ void __launch_bounds__(LF_THREADS) latent_fold_kernel(const float* __restrict__ part, const float* __restrict__ sink,
                                                                 float* __restrict__ ctx, const int* __restrict__ positions,
                                                                 int n_tokens, int H, int R, int run_keys, int n_runs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float wts[LF_MAX_RUNS];
    __shared__ float inv_s;
    const int lane = threadIdx.x & 31;
    const long long w = blockIdx.x;
    const int t = (int)(w / H), head = (int)(w % H);
    const int used = min(n_runs, positions[t] / run_keys + 1);               // runs that hold keys of this query
    const size_t stride = (size_t)R + 2;
    const float* p = part + (size_t)w * n_runs * stride;
    if (threadIdx.x < 32) {
        const float sk = sink ? sink[head] : -INFINITY;
        float mf = sk;
        for (int r = lane; r < used; r += 32) mf = fmaxf(mf, p[r * stride]);
        mf = warp_max(mf);
        float l = 0.f;
        for (int r = lane; r < used; r += 32) {
            const float wr = expf(p[r * stride] - mf);
            wts[r] = wr;
            l = fmaf(p[r * stride + 1], wr, l);
        }
        l = warp_sum(l);
        if (sink) l += expf(sk - mf);
        if (lane == 0) inv_s = 1.0f / l;
    }
    __syncthreads();
    const float inv = inv_s;
    float* o = ctx + (size_t)w * R;
    for (int d = threadIdx.x; d < R; d += LF_THREADS) {
        const float* pd = p + 2 + d;
        float s = 0.f;
        int r = 0;
        for (; r + 8 <= used; r += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = pd[(r + i) * stride];
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(v[i], wts[r + i], s);
        }
        for (; r < used; ++r) s = fmaf(pd[r * stride], wts[r], s);
        o[d] = s * inv;
    }
}

extern "C" int idm_latent_attention_max_rank() { return 1024; }

static bool latent_mma_fits(int R, int D) {
#if defined(IDM_BF16)
    static const int on = idm_pdl_flag("IDM_LATENT_MMA", 1);       // IDM_LATENT_MMA=0: the kernel of plain 32-bit sums everywhere
    return on && D % 16 == 0 && R % 32 == 0 && R <= 512;
#else
    return false;
#endif
}
// heads a block of the attention kernel has (what the host spreads a step's runs by): 16 on tensor-core fragments,
// else 8 warps of one head each, or of two where the layer has more than 8 heads
extern "C" int idm_latent_attention_heads_per_block(int H, int R, int D) {
    return latent_mma_fits(R, D) ? 16 : (H > LA_WARPS ? 2 * LA_WARPS : LA_WARPS);
}

// run_keys: a multiple of 32; n_runs * run_keys covers every position of the step (n_runs == 1: no scratch)
extern "C" int idm_latent_attention(const float* qa, const void* pool, const int* table, int table_stride,
                                    const int* token_seq, const int* positions, const int* slots, const float* sink,
                                    float* ctx, float* part, int n_tokens, int H, int R, int D, float scale,
                                    int run_keys, int n_runs, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && R > 0 && D >= R && R <= 1024, "latent_attention: heads=%d rank=%d row=%d (rank at most 1024)", H, R, D);
    IDM_REQUIRE(n_runs >= 1 && n_runs <= LF_MAX_RUNS && run_keys > 0 && run_keys % 32 == 0 && (n_runs == 1 || part != nullptr),
                "latent_attention: %d runs of %d keys (at most %d runs)", n_runs, run_keys, LF_MAX_RUNS);
    LatentArgs a;
    a.qa = qa; a.pool = (const T*)pool; a.table = table; a.table_stride = table_stride;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.sink = sink; a.ctx = ctx; a.part = part;
    a.n_tokens = n_tokens; a.H = H; a.R = R; a.D = D; a.scale = scale; a.run_keys = run_keys; a.n_runs = n_runs;
#if defined(IDM_BF16)
    if (idm_latent_attention_heads_per_block(H, R, D) == 16 && latent_mma_fits(R, D)) {
        int units = D / 8;                                  // rows of 16 bytes x an odd number: no bank is hit twice by a fragment load
        if (units % 2 == 0) ++units;
        a.stride_words = units * 4;
        a.n_buf = 2;
        const size_t smem = ((size_t)(16 + 64) * units * 8 + 16 * 40) * 2 + 2 * LM_WARPS * 16 * sizeof(float);
        const dim3 grid(n_tokens, (H + 15) / 16, n_runs);
        IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "latent_attention: grid %d x %d", grid.y, grid.z);
#define LM_LAUNCH(NT)                                                                                                    \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(latent_attention_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        idm_launch(latent_attention_mma_kernel<NT>, grid, dim3(LM_WARPS * 32), smem, stream, a);                         \
    } while (0)
        if (R <= 128) LM_LAUNCH(4);
        else if (R <= 256) LM_LAUNCH(8);
        else LM_LAUNCH(16);
#undef LM_LAUNCH
        IDM_LAUNCH_CHECK("latent_attention_mma");
        if (n_runs > 1) {
            idm_launch(latent_fold_kernel, dim3((unsigned)(n_tokens * H)), dim3(LF_THREADS), 0, stream, (const float*)part, sink, ctx,
                       positions, n_tokens, H, R, run_keys, n_runs);
            IDM_LAUNCH_CHECK("latent_fold");
        }
        return 0;
    }
#endif
    // a row of the staged block: whole 16-byte pieces, and a stride of 4 (mod 8) words, so that eight lanes that
    // read 16 bytes each at the same column of eight rows touch every bank once
    int words = (D * (int)sizeof(T) + 15) / 16 * 4;
    while (words % 8 != 4) words += 4;
    a.stride_words = words;
    // two staging buffers (the next block of keys on its way while this one is scored) where they fit
    const int hpw = H > LA_WARPS ? 2 : 1;                  // heads of a warp
    const size_t q_bytes = (size_t)LA_WARPS * hpw * ((D + 3) & ~3) * sizeof(float), tile_bytes = (size_t)32 * words * 4;
    a.n_buf = q_bytes + 2 * tile_bytes <= 200 * 1024 ? 2 : 1;
    const size_t smem = q_bytes + a.n_buf * tile_bytes;
    IDM_REQUIRE(smem <= 220 * 1024, "latent_attention: rows of %d do not fit shared memory", D);
    const dim3 grid(n_tokens, (H + LA_WARPS * hpw - 1) / (LA_WARPS * hpw), n_runs);
    IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "latent_attention: grid %d x %d", grid.y, grid.z);
#define LA_LAUNCH_H(NACC, HPW)                                                                                           \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(latent_attention_kernel<NACC, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        idm_launch(latent_attention_kernel<NACC, HPW>, grid, dim3(LA_WARPS * 32), smem, stream, a);                      \
    } while (0)
#define LA_LAUNCH(NACC)                                                                                                  \
    do { if (hpw == 2) LA_LAUNCH_H(NACC, 2); else LA_LAUNCH_H(NACC, 1); } while (0)
    if (R <= 64) LA_LAUNCH(2);
    else if (R <= 128) LA_LAUNCH(4);
    else if (R <= 256) LA_LAUNCH(8);
    else if (R <= 512) LA_LAUNCH(16);
    else LA_LAUNCH(32);
#undef LA_LAUNCH
#undef LA_LAUNCH_H
    IDM_LAUNCH_CHECK("latent_attention");
    if (n_runs > 1) {
        idm_launch(latent_fold_kernel, dim3((unsigned)(n_tokens * H)), dim3(LF_THREADS), 0, stream, (const float*)part, sink, ctx,
                   positions, n_tokens, H, R, run_keys, n_runs);
        IDM_LAUNCH_CHECK("latent_fold");
    }
    return 0;
}

// ------------------------------------------------------------------ whole prompts: keys and values per head
// A step that brings whole prompts (every sequence from its first token) has more queries than heads' worth of
// latent space pays for: there the keys and values are made per head from the step's rows once, k_h = [Uk_h c | r]
// and v_h = Uv_h c, and the step runs the attention kernel for heads with keys and values of their own.  This
// kernel lays its operands out: q [N, H, hd] = [qn | turn(qr) | 0], and pages of their own [pages, H, PAGE, hd]
// for k and v (0 behind a head's own dims), addressed through a block table of the step's own.
// proj: the joint projection (a head's query at column h * (dn + dr)); up: [N, H * dn + H * dv] = the rows' c times
// [Uk ; Uv]; rows: the step's packed [c | r] rows in the storage type.  One block per token.
__global__ void __launch_bounds__(256) latent_expand_pack_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ up,
                                                                 const T* __restrict__ rows, int H, int dn, int dr, int dv, int R,
                                                                 int rot_dims, const float2* __restrict__ cs, int half, float mag,
                                                                 int hd, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                                 const int* __restrict__ table, int table_stride,
                                                                 const int* __restrict__ token_seq, const int* __restrict__ positions,
                                                                 const int* __restrict__ slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t], slot = slots[token_seq[t]];
    const int page = table[(size_t)slot * table_stride + pos / IDM_PAGE];
    const float* pq = proj + (size_t)t * ld;
    const float* pu = up + (size_t)t * (size_t)(H * dn + H * dv);
    const T* r = rows + (size_t)t * (R + dr) + R;
    for (int e = threadIdx.x; e < H * hd; e += blockDim.x) {
        const int h = e / hd, d = e % hd;
        float qv = 0.f;
        T kk, vv;
        from_f32(kk, 0.f); from_f32(vv, 0.f);
        if (d < dn) {
            qv = pq[h * (dn + dr) + d];
            from_f32(kk, pu[h * dn + d]);
        } else if (d < dn + dr) {
            const int j = d - dn;
            const float* qr = pq + h * (dn + dr) + dn;
            qv = qr[j];
            if ((j | 1) < rot_dims) {                       // the pair (j & ~1, j | 1) is turned
                const float2 a = cs[(size_t)t * half + (j >> 1)];
                const float co = a.x * mag, si = a.y * mag;
                qv = (j & 1) ? qr[j] * co + qr[j - 1] * si : qr[j] * co - qr[j + 1] * si;
            }
            kk = r[j];
        }
        if (d < dv) from_f32(vv, pu[H * dn + h * dv + d]);
        from_f32(q[((size_t)t * H + h) * hd + d], qv);
        const size_t at = (((size_t)page * H + h) * IDM_PAGE + pos % IDM_PAGE) * hd + d;
        k[at] = kk;
        v[at] = vv;
    }
}

extern "C" int idm_latent_expand_pack(const float* proj, int ld, const float* up, const void* rows, int H, int dn, int dr,
                                      int dv, int R, int rot_dims, const float* cs, int half, float mag, int hd, void* q,
                                      void* k, void* v, const int* table, int table_stride, const int* token_seq,
                                      const int* positions, const int* slots, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && dv > 0 && dn + dr <= hd && dv <= hd, "latent_expand_pack: heads of %d + %d and %d in %d",
                dn, dr, dv, hd);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "latent_expand_pack: %d turned dims of %d with a table of %d angles", rot_dims, dr, half);
    idm_launch(latent_expand_pack_kernel, dim3(n_tokens), dim3(256), 0, stream, proj, ld, up, (const T*)rows, H, dn, dr, dv, R, rot_dims,
               (const float2*)cs, half, mag, hd, (T*)q, (T*)k, (T*)v, table, table_stride, token_seq, positions, slots);
    IDM_LAUNCH_CHECK("latent_expand_pack");
    return 0;
}
