// A matrix state per head that decays by ONE factor per token and head:
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T          (S: dk x dv; a_t, b_t scalars of the token and head)
//     o_t = S_t^T q_t  (+ skip_h v_t)
//
// which is the recurrence of a selective state space layer (a_t = e^(A dt_t), b_t = dt_t, k = B, q = C,
// v = x, skip = D) and of a matrix memory with exponential gates (a_t = e^(f_t + m_(t-1) - m_t),
// b_t = e^(i_t - m_t), m the running maximum of the log gates).  The matrix memory also keeps a
// normalizer n_t = a_t n_(t-1) + b_t k_t, stored as one more value column of the state, and divides:
// o_t <- o_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).
//
// The state lives in 32-bit floats per sequence slot, [slot][head][dv (+1)][dk]; log a_t and b_t come as
// 32-bit numbers per token and head; q, k, v are 32-bit rows (any row stride, any column offset); several
// heads may share one q and k (a group).  Everything is computed in 32-bit.
//
// Work of the token-by-token kernel: a block is (16 value columns, head, sequence) and walks the
// sequence's tokens in order; a value column is owned by 8 lanes, lane p holding rows p, p+8, ... of that
// column in registers.  With a normalizer every block carries that column too (as a 17th group of lanes),
// so that it can divide without waiting for another block; the block of the first tile stores it.  The
// order of every sum depends on nothing but dk, so a prompt gives the same numbers however it is cut.
#include "common.cuh"

#define SS_COLS 16
#define SS_PART 8
#define SS_CHUNK 8

template <int R>
__global__ void __launch_bounds__(SS_COLS * SS_PART + 32)
scalar_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                   const float* __restrict__ v, int ldv, const float* __restrict__ log_a, int ld_a,
                   const float* __restrict__ b_in, int ld_b, const float* __restrict__ skip,
                   const float* __restrict__ m_tok, float q_scale, float* __restrict__ state,
                   const int* __restrict__ slots, const int* __restrict__ cu, float* __restrict__ o, int n_heads,
                   int heads_per_group, int dk, int dv, int normalizer) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    float* qs = smem;                           // [SS_CHUNK][dk]
    float* ks = qs + SS_CHUNK * dk;             // [SS_CHUNK][dk], already times b_t
    float* vs = ks + SS_CHUNK * dk;             // [SS_CHUNK][SS_COLS]
    float* as = vs + SS_CHUNK * SS_COLS;        // [SS_CHUNK] decay factors
    float* ms = as + SS_CHUNK;                  // [SS_CHUNK] e^(-m_t)
    float* acc_s = ms + SS_CHUNK;               // [SS_CHUNK][SS_COLS + 1]
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, p = tid & (SS_PART - 1), jl = tid >> 3;
    const int n_threads = blockDim.x;
    const bool is_n = jl == SS_COLS;                          // the normalizer's lanes
    const int cols = dv + (normalizer ? 1 : 0);
    const int j = jl >= SS_COLS ? dv : tile * SS_COLS + jl;
    const bool live = is_n ? normalizer != 0 : (jl < SS_COLS && j < dv);    // a whole last warp: its other lanes idle
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const int slot = mv_read_slot(slots[b]);
    const size_t qk_off = (size_t)(h / heads_per_group) * dk;
    float* srow = state + (((size_t)slot * n_heads + h) * cols + (live ? j : 0)) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = p + SS_PART * r;
        S[r] = (live && i < dk) ? srow[i] : 0.f;
    }
    const float sk = skip ? skip[h] : 0.f;
    for (int c0 = 0; c0 < len; c0 += SS_CHUNK) {
        const int nt = min(SS_CHUNK, len - c0);
        __syncthreads();
        if (tid < nt) {
            const size_t row = (size_t)(row0 + c0 + tid);
            as[tid] = expf(log_a[row * ld_a + h]);
            ms[tid] = m_tok ? expf(-m_tok[row * n_heads + h]) : 0.f;
        }
        for (int idx = tid; idx < nt * dk; idx += n_threads) {
            const int t = idx / dk, i = idx - t * dk;
            const size_t row = (size_t)(row0 + c0 + t);
            qs[idx] = q[row * ldq + qk_off + i] * q_scale;
            ks[idx] = k[row * ldk + qk_off + i] * b_in[row * ld_b + h];
        }
        for (int idx = tid; idx < nt * SS_COLS; idx += n_threads) {
            const int t = idx / SS_COLS, c = idx - t * SS_COLS, col = tile * SS_COLS + c;
            vs[idx] = col < dv ? v[(size_t)(row0 + c0 + t) * ldv + (size_t)h * dv + col] : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = is_n ? 1.f : vs[t * SS_COLS + (jl < SS_COLS ? jl : 0)];
            const float a = as[t];
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + SS_PART * r;
                if (i < dk) {
                    S[r] = fmaf(a, S[r], kt[i] * vj);
                    acc = fmaf(S[r], qt[i], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (p == 0 && jl <= SS_COLS) acc_s[t * (SS_COLS + 1) + jl] = acc + (is_n ? 0.f : sk * vj);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * SS_COLS; idx += n_threads) {
            const int t = idx / SS_COLS, c = idx - t * SS_COLS, col = tile * SS_COLS + c;
            if (col >= dv) continue;
            float val = acc_s[t * (SS_COLS + 1) + c];
            if (normalizer) val = val / (fmaxf(fabsf(acc_s[t * (SS_COLS + 1) + SS_COLS]), ms[t]) + 1e-6f);
            o[(size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv + col] = val;
        }
    }
    if (live && (!is_n || tile == 0) && mv_slot_ok(slots[b])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = p + SS_PART * r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

MV_GUARD_SETTER(scalar_scan)

// q, k [N, >= (n_heads / heads_per_group) * dk], v [N, >= n_heads * dv] with row strides (elements);
// log_a, b [N, >= n_heads] with row strides; skip [n_heads] or null; m_tok [N, n_heads] dense or null
// (needed with a normalizer); state [slots][n_heads][dv + normalizer][dk]; o [N, n_heads * dv] dense.
MV_API int mv_scalar_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                          const float* log_a, int ld_a, const float* b, int ld_b, const float* skip,
                          const float* m_tok, float q_scale, float* state, const int* slots, const int* cu, float* o,
                          int n_seqs, int n_heads, int heads_per_group, int dk, int dv, int normalizer,
                          cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || heads_per_group < 1 || n_heads % heads_per_group || (normalizer && !m_tok))
        return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + SS_COLS - 1) / SS_COLS, n_heads, n_seqs);
    const int threads = SS_COLS * SS_PART + (normalizer ? 32 : 0);
    const size_t smem = sizeof(float) * ((size_t)SS_CHUNK * (2 * dk + SS_COLS + 2 + SS_COLS + 1));
#define SS_LAUNCH(R)                                                                                              \
    mv_launch(scalar_scan_kernel<R>, grid, threads, smem, stream, q, ldq, k, ldk, v, ldv, log_a, ld_a, b, ld_b,  \
              skip, m_tok, q_scale, state, slots, cu, o, n_heads, heads_per_group, dk, dv, normalizer)
    if (dk <= 64) SS_LAUNCH(8);
    else if (dk <= 128) SS_LAUNCH(16);
    else SS_LAUNCH(32);
#undef SS_LAUNCH
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// The log gates of a matrix memory and their running maximum, per sequence and head:
//     i_t = cap tanh((zi_t + bi) / cap),  f_t = log sigmoid(cap tanh((zf_t + bf) / cap)),
//     m_t = max(f_t + m_(t-1), i_t)   (m before a sequence's first token is 0: a zeroed state),
//     log a_t = f_t + m_(t-1) - m_t,  b_t = e^(i_t - m_t).
// The step m -> max(m + f, i) composes: first (f1, i1), then (f2, i2) is m -> max(m + f1 + f2, max(i1 + f2, i2)).
// A warp is one (sequence, head): it takes 32 tokens at a time, a lane a token, scans the pairs with that rule
// (five shuffles) and hands the last maximum on to the next 32.  A step of one token a sequence is the rule itself.
// m is kept per slot and head.
__device__ __forceinline__ float ss_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

__global__ void __launch_bounds__(128)
memory_gates_kernel(const float* __restrict__ zi, int ld_i, const float* __restrict__ zf, int ld_f,
                    const float* __restrict__ bi, const float* __restrict__ bf, float cap, float* __restrict__ m_state,
                    const int* __restrict__ slots, const int* __restrict__ cu, float* __restrict__ log_a,
                    float* __restrict__ b_out, float* __restrict__ m_tok, int n_seqs, int n_heads) {
    mv_pdl_begin();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp >= n_seqs * n_heads) return;
    const int b = warp / n_heads, h = warp - b * n_heads;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const float inv_cap = 1.0f / cap;
    const int slot = mv_read_slot(slots[b]);
    float m = m_state[(size_t)slot * n_heads + h];
    const float bih = bi[h], bfh = bf[h];
    for (int t0 = 0; t0 < len; t0 += 32) {
        const int t = t0 + lane;
        const bool in = t < len;
        const size_t row = (size_t)(row0 + (in ? t : 0));
        const float il = in ? cap * tanhf((zi[row * ld_i + h] + bih) * inv_cap) : -INFINITY;
        const float fl = in ? ss_log_sigmoid(cap * tanhf((zf[row * ld_f + h] + bfh) * inv_cap)) : 0.f;
        float A = fl, B = il;                         // the tokens up to this lane's as one step m -> max(m + A, B)
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float a_up = __shfl_up_sync(0xffffffffu, A, d), b_up = __shfl_up_sync(0xffffffffu, B, d);
            if (lane >= d) {
                B = fmaxf(b_up + A, B);
                A = a_up + A;
            }
        }
        const float m_t = fmaxf(m + A, B);
        float m_before = __shfl_up_sync(0xffffffffu, m_t, 1);
        if (lane == 0) m_before = m;
        if (in) {
            const size_t at = row * n_heads + h;
            log_a[at] = fl + m_before - m_t;
            b_out[at] = expf(il - m_t);
            m_tok[at] = m_t;
        }
        m = __shfl_sync(0xffffffffu, m_t, min(31, len - t0 - 1));
    }
    if (lane == 0 && mv_slot_ok(slots[b])) m_state[(size_t)slot * n_heads + h] = m;
}

// zi, zf: the gates' projections [N, >= n_heads] with row strides; bi, bf [n_heads]; m_state [slots][n_heads];
// log_a, b_out, m_tok [N, n_heads] dense.
MV_API int mv_memory_gates(const float* zi, int ld_i, const float* zf, int ld_f, const float* bi, const float* bf,
                           float cap, float* m_state, const int* slots, const int* cu, float* log_a, float* b_out,
                           float* m_tok, int n_seqs, int n_heads, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!(cap > 0.f) || n_heads < 1) return (int)cudaErrorInvalidValue;
    const int warps = n_seqs * n_heads;
    mv_launch(memory_gates_kernel, (warps + 3) / 4, 128, 0, stream, zi, ld_i, zf, ld_f, bi, bf, cap, m_state, slots, cu, log_a,
              b_out, m_tok, n_seqs, n_heads);
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// The same recurrence for steps that bring many tokens a sequence, in chunks of SC_CHUNK tokens.  With c_t the
// sum of log a over the chunk's tokens up to t (all of it <= 0) and S0 the state before the chunk,
//
//     o_t   = e^(c_t) q_t^T S0 + sum_{s <= t} (q_t . k_s) e^(c_t - c_s) b_s v_s  (+ skip v_t),
//     S_end = e^(c_last) S0 + sum_s e^(c_last - c_s) b_s k_s v_s^T.
//
// Every exponent is a difference of cumulative logarithms taken the right way round, so every factor lies in
// (0, 1] (times b): nothing overflows however small a decay is.  Because the decay is one number a head, q and k
// need no decayed copies: the products q_t . k_s are worked out once per GROUP of heads that share q and k (the
// first kernel), and each head puts its own factors on them.  The second kernel walks a sequence's chunks with
// the state in registers: a block is 16 value columns of one head of one sequence, its 32 half-warps each hold
// RH key channels of every column.  With a normalizer the state's last column is fed ones instead of values and
// comes out as n . q; a third kernel divides.  All of it is float32 on the CUDA cores.
//
// Chunks are numbered floor(cu[b] / SC_CHUNK) + b + c for chunk c of the step's sequence b: distinct numbers
// below N / SC_CHUNK + n_seqs + 1 that need nothing from the host.
#define SC_CHUNK 32
#define SC_COLS 16
#define SC_THREADS 256
#define SC_SCAN_THREADS 512
#define SC_GROUPS (SC_SCAN_THREADS / 16)
#define SC_RED_STRIDE (SC_CHUNK * SC_COLS + 16)

__global__ void __launch_bounds__(SC_THREADS)
scalar_chunk_products_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                             const int* __restrict__ cu, float* __restrict__ G, int n_groups, int dk) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    const int lds = dk + 1;                         // odd row stride: rows of different tokens fall into different banks
    float* qa = smem;                               // [SC_CHUNK][lds]
    float* ka = qa + SC_CHUNK * lds;
    const int c = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (c * SC_CHUNK >= len) return;
    const int nt = min(SC_CHUNK, len - c * SC_CHUNK);
    const int first = row0 + c * SC_CHUNK;
    const int chunk = row0 / SC_CHUNK + b + c;
    for (int idx = threadIdx.x; idx < nt * dk; idx += SC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        qa[t * lds + i] = q[(size_t)(first + t) * ldq + (size_t)g * dk + i];
        ka[t * lds + i] = k[(size_t)(first + t) * ldk + (size_t)g * dk + i];
    }
    __syncthreads();
    float* Gc = G + ((size_t)chunk * n_groups + g) * SC_CHUNK * SC_CHUNK;
    for (int p = threadIdx.x; p < SC_CHUNK * SC_CHUNK; p += SC_THREADS) {
        const int t = p / SC_CHUNK, s = p - t * SC_CHUNK;
        float sum = 0.f;
        if (s <= t && t < nt) {
            const float* qt = qa + t * lds;
            const float* kt = ka + s * lds;
            for (int i = 0; i < dk; ++i) sum = fmaf(qt[i], kt[i], sum);
        }
        Gc[p] = sum;
    }
}

template <int RH>
__global__ void __launch_bounds__(SC_SCAN_THREADS)
scalar_chunk_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                         const float* __restrict__ v, int ldv, const float* __restrict__ log_a, int ld_a,
                         const float* __restrict__ b_in, int ld_b, const float* __restrict__ skip, float q_scale,
                         const float* __restrict__ G, float* __restrict__ state, const int* __restrict__ slots,
                         const int* __restrict__ cu, float* __restrict__ o, int n_heads, int heads_per_group, int dk,
                         int dv, int ones_col) {
    mv_pdl_begin();
    constexpr int DKP = SC_GROUPS * RH;
    extern __shared__ __align__(16) float smem[];
    float* qt = smem;                               // [SC_CHUNK][DKP], zero beyond dk
    float* kt = qt + SC_CHUNK * DKP;
    float* vt = kt + SC_CHUNK * DKP;                // [SC_CHUNK][SC_COLS]
    float* pt = vt + SC_CHUNK * SC_COLS;            // [SC_CHUNK][SC_CHUNK]
    float* la = pt + SC_CHUNK * SC_CHUNK;           // [SC_CHUNK] log decays, then their running sum
    float* bs = la + SC_CHUNK;                      // [SC_CHUNK] input factors
    float* e1 = bs + SC_CHUNK;                      // [SC_CHUNK] e^(c_t) q_scale
    float* e2 = e1 + SC_CHUNK;                      // [SC_CHUNK] e^(c_last - c_t) b_t
    float* el = e2 + SC_CHUNK;                      // [1] e^(c_last) (padded to 16 floats)
    float* red = el + 16;                           // [SC_GROUPS][SC_RED_STRIDE]: [SC_CHUNK][SC_COLS] a group
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, col = tid & 15, grp = tid >> 4;
    const int cols = dv + (ones_col >= 0 ? 1 : 0);  // the state's and the output's columns
    const int j = tile * SC_COLS + col;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const int slot = mv_read_slot(slots[b]);
    const int n_groups = n_heads / heads_per_group, g = h / heads_per_group;
    const size_t goff = (size_t)g * dk;
    float* srow = state + (((size_t)slot * n_heads + h) * cols + (j < cols ? j : 0)) * dk;
    float S[RH];
#pragma unroll
    for (int r = 0; r < RH; ++r) {
        const int i = grp * RH + r;
        S[r] = (j < cols && i < dk) ? srow[i] : 0.f;
    }
    const float sk = skip ? skip[h] : 0.f;
    const int n_chunks = (len + SC_CHUNK - 1) / SC_CHUNK;
    constexpr int IT = SC_CHUNK * DKP / SC_SCAN_THREADS;
    static_assert(SC_CHUNK * SC_COLS == SC_SCAN_THREADS && SC_CHUNK * SC_CHUNK % SC_SCAN_THREADS == 0,
                  "a thread requests one value of v and whole rounds of the products");
    float rq[IT], rk[IT], rv, rp[SC_CHUNK * SC_CHUNK / SC_SCAN_THREADS], rla = 0.f, rb = 0.f;
    auto request = [&](int c) {
        const int nt = min(SC_CHUNK, len - c * SC_CHUNK);
        const int first = row0 + c * SC_CHUNK;
        const int chunk = row0 / SC_CHUNK + b + c;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int idx = tid + it * SC_SCAN_THREADS, t = idx / DKP, i = idx - t * DKP;
            const bool in = t < nt && i < dk;
            rq[it] = in ? q[(size_t)(first + t) * ldq + goff + i] : 0.f;
            rk[it] = in ? k[(size_t)(first + t) * ldk + goff + i] : 0.f;
        }
        {
            const int t = tid / SC_COLS, cc = tile * SC_COLS + (tid - t * SC_COLS);
            rv = t < nt ? (cc < dv ? v[(size_t)(first + t) * ldv + (size_t)h * dv + cc] : (cc == ones_col ? 1.f : 0.f)) : 0.f;
        }
        const float* Gc = G + ((size_t)chunk * n_groups + g) * SC_CHUNK * SC_CHUNK;
#pragma unroll
        for (int it = 0; it < SC_CHUNK * SC_CHUNK / SC_SCAN_THREADS; ++it) rp[it] = Gc[tid + it * SC_SCAN_THREADS];
        if (tid < SC_CHUNK) {
            rla = tid < nt ? log_a[(size_t)(first + tid) * ld_a + h] : 0.f;
            rb = tid < nt ? b_in[(size_t)(first + tid) * ld_b + h] : 0.f;
        }
    };
    request(0);
    for (int c = 0; c < n_chunks; ++c) {
        const int nt = min(SC_CHUNK, len - c * SC_CHUNK);
        const int first = row0 + c * SC_CHUNK;
        __syncthreads();                            // the chunk before is done with shared memory
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            qt[tid + it * SC_SCAN_THREADS] = rq[it];
            kt[tid + it * SC_SCAN_THREADS] = rk[it];
        }
        vt[tid] = rv;
#pragma unroll
        for (int it = 0; it < SC_CHUNK * SC_CHUNK / SC_SCAN_THREADS; ++it) pt[tid + it * SC_SCAN_THREADS] = rp[it];
        if (tid < SC_CHUNK) {
            // the running sum of the log decays over the chunk (one warp), and the factors that follow from it
            float run = rla;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, run, d);
                if (tid >= d) run += up;
            }
            const float last = __shfl_sync(0xffffffffu, run, nt - 1);
            la[tid] = run;
            bs[tid] = rb;
            e1[tid] = expf(run) * q_scale;
            e2[tid] = tid < nt ? expf(last - run) * rb : 0.f;
            if (tid == 0) el[0] = expf(last);
        }
        __syncthreads();
        if (c + 1 < n_chunks) request(c + 1);
        // this head's factors on the group's products: e^(c_t - c_s) b_s q_scale (own entries only: no one else reads them yet)
#pragma unroll
        for (int it = 0; it < SC_CHUNK * SC_CHUNK / SC_SCAN_THREADS; ++it) {
            const int p = tid + it * SC_SCAN_THREADS, t = p / SC_CHUNK, s = p - t * SC_CHUNK;
            pt[p] = (s <= t && t < nt) ? pt[p] * expf(la[t] - la[s]) * bs[s] * q_scale : 0.f;
        }
        // what the chunk's tokens read from the state before the chunk: this half-warp's key channels
#pragma unroll 4
        for (int t = 0; t < SC_CHUNK; ++t) {
            const float4* q4 = reinterpret_cast<const float4*>(qt + t * DKP + grp * RH);
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RH; r += 4) {
                const float4 x = q4[r >> 2];
                acc = fmaf(x.x, S[r], acc); acc = fmaf(x.y, S[r + 1], acc);
                acc = fmaf(x.z, S[r + 2], acc); acc = fmaf(x.w, S[r + 3], acc);
            }
            red[grp * SC_RED_STRIDE + t * SC_COLS + col] = acc;
        }
        // the state after the chunk
        const float decay = el[0];
#pragma unroll
        for (int r = 0; r < RH; ++r) S[r] *= decay;
#pragma unroll 4
        for (int s = 0; s < SC_CHUNK; ++s) {
            const float vj = vt[s * SC_COLS + col] * e2[s];
            const float4* k4 = reinterpret_cast<const float4*>(kt + s * DKP + grp * RH);
#pragma unroll
            for (int r = 0; r < RH; r += 4) {
                const float4 x = k4[r >> 2];
                S[r] = fmaf(x.x, vj, S[r]); S[r + 1] = fmaf(x.y, vj, S[r + 1]);
                S[r + 2] = fmaf(x.z, vj, S[r + 2]); S[r + 3] = fmaf(x.w, vj, S[r + 3]);
            }
        }
        __syncthreads();
        // outputs: the groups' shares in a fixed order, then the chunk's own tokens
        for (int idx = tid; idx < nt * SC_COLS; idx += SC_SCAN_THREADS) {
            const int t = idx / SC_COLS, cc = idx - t * SC_COLS;
            float sum = 0.f;
#pragma unroll
            for (int gg = 0; gg < SC_GROUPS; ++gg) sum += red[gg * SC_RED_STRIDE + t * SC_COLS + cc];
            sum *= e1[t];
            for (int s = 0; s <= t; ++s) sum = fmaf(pt[t * SC_CHUNK + s], vt[s * SC_COLS + cc], sum);
            const int oc = tile * SC_COLS + cc;
            if (oc < dv) sum = fmaf(sk, vt[t * SC_COLS + cc], sum);
            if (oc < cols) o[(size_t)(first + t) * n_heads * cols + (size_t)h * cols + oc] = sum;
        }
    }
    if (j < cols && mv_slot_ok(slots[b])) {
#pragma unroll
        for (int r = 0; r < RH; ++r) {
            const int i = grp * RH + r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

template <int RH>
static int scalar_chunk_scan_launch(dim3 grid, cudaStream_t stream, const float* q, int ldq, const float* k, int ldk,
                                    const float* v, int ldv, const float* log_a, int ld_a, const float* b, int ld_b,
                                    const float* skip, float q_scale, const float* G, float* state, const int* slots,
                                    const int* cu, float* o, int n_heads, int hpg, int dk, int dv, int ones_col) {
    const size_t smem = sizeof(float) * ((size_t)2 * SC_CHUNK * SC_GROUPS * RH + SC_CHUNK * SC_COLS + SC_CHUNK * SC_CHUNK +
                                         4 * SC_CHUNK + 16 + SC_GROUPS * SC_RED_STRIDE);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(scalar_chunk_scan_kernel<RH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    mv_launch(scalar_chunk_scan_kernel<RH>, grid, SC_SCAN_THREADS, smem, stream, q, ldq, k, ldk, v, ldv, log_a, ld_a, b, ld_b,
              skip, q_scale, G, state, slots, cu, o, n_heads, hpg, dk, dv, ones_col);
    return mv_launch_status();
}

// o[n, h, :] = o_aug[n, h, :dv] / (max(|o_aug[n, h, dv]|, e^(-m[n, h])) + 1e-6)
__global__ void __launch_bounds__(256)
memory_normalize_kernel(const float* __restrict__ o_aug, const float* __restrict__ m_tok, float* __restrict__ o,
                        long long total, int dv) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long nh = idx / dv;
    const int d = (int)(idx - nh * dv);
    const float den = fmaxf(fabsf(o_aug[nh * (dv + 1) + dv]), expf(-m_tok[nh])) + 1e-6f;
    o[idx] = o_aug[nh * (dv + 1) + d] / den;
}

// How many chunks the scratch of a step of N tokens in n_seqs sequences must hold.
MV_API int mv_scalar_chunks(int N, int n_seqs) { return N / SC_CHUNK + n_seqs + 1; }

// Arguments as mv_scalar_scan, plus the longest sequence's tokens (max_len) and scratch: G [chunks, groups,
// SC_CHUNK, SC_CHUNK] with chunks = mv_scalar_chunks(N, n_seqs), and with a normalizer o_aug [N, n_heads * (dv + 1)].
MV_API int mv_scalar_scan_chunked(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                  const float* log_a, int ld_a, const float* b, int ld_b, const float* skip,
                                  const float* m_tok, float q_scale, float* state, const int* slots, const int* cu,
                                  float* o, float* G, float* o_aug, int N, int n_seqs, int max_len, int n_heads,
                                  int heads_per_group, int dk, int dv, int normalizer, cudaStream_t stream) {
    if (n_seqs <= 0 || max_len <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || heads_per_group < 1 || n_heads % heads_per_group ||
        (normalizer && (!m_tok || !o_aug)))
        return (int)cudaErrorInvalidValue;
    const int n_groups = n_heads / heads_per_group;
    const size_t smem_a = sizeof(float) * (size_t)2 * SC_CHUNK * (dk + 1);
    static size_t attr_a = 0;
    if (smem_a > attr_a) {
        cudaFuncSetAttribute(scalar_chunk_products_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        attr_a = smem_a;
    }
    mv_launch(scalar_chunk_products_kernel, dim3((max_len + SC_CHUNK - 1) / SC_CHUNK, n_groups, n_seqs), SC_THREADS, smem_a,
              stream, q, ldq, k, ldk, cu, G, n_groups, dk);
    int code = mv_launch_status();
    if (code) return code;
    const int cols = dv + (normalizer ? 1 : 0);
    const dim3 grid((cols + SC_COLS - 1) / SC_COLS, n_heads, n_seqs);
    float* out = normalizer ? o_aug : o;
    const int ones_col = normalizer ? dv : -1;
    if (dk <= 128)
        code = scalar_chunk_scan_launch<4>(grid, stream, q, ldq, k, ldk, v, ldv, log_a, ld_a, b, ld_b, skip, q_scale, G, state,
                                           slots, cu, out, n_heads, heads_per_group, dk, dv, ones_col);
    else
        code = scalar_chunk_scan_launch<8>(grid, stream, q, ldq, k, ldk, v, ldv, log_a, ld_a, b, ld_b, skip, q_scale, G, state,
                                           slots, cu, out, n_heads, heads_per_group, dk, dv, ones_col);
    if (code || !normalizer) return code;
    const long long total = (long long)N * n_heads * dv;
    mv_launch(memory_normalize_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, (const float*)o_aug, m_tok, o, total, dv);
    return mv_launch_status();
}
