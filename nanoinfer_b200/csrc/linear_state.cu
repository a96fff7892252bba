// Mixers whose memory is a matrix per head that decays and takes one outer product per token, over a flat batch of
// requests (each brings a prompt's portion or one decoded token), and the small kernels around them. A request's
// state is a row of 32-bit floats in a slot of a state tensor (row stride `state_ld`, the part of one mechanism starts
// at a column offset); which request owns which rows and which slot is read from device arrays (q_start, req_index,
// slots), so a captured graph can replay the launches for other requests. Every kernel walks a request's tokens with
// the same arithmetic per token whatever the cut, and nothing depends on what else is in the batch.
//
//  * linear_state_scan:  S_t = diag(w_t) S_(t-1) + k_t v_t^T per head (S: key channel x value channel), read after the
//    update (o_t = S_t^T q_t) or, with a bonus u, before it (o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t). The decay is a
//    vector per key channel or one number per head; q and k may be shared by groups of heads; v may carry a factor per
//    (token, head). Gated linear attention, a time mix with bonus and a state-space mixer with scalar decays are this
//    walk with different inputs.
//  * conv_tokens / conv_tail: a short causal convolution per channel whose last taps-1 inputs are kept in the state.
//  * token_shift: blends of every token with the token before it (the request's last token is kept in the state).
//  * decay_map, step_sizes: the decays, rounded to 32 bits once from 64-bit exponentials (a decay is raised to hundreds
//    of powers along a sequence).
#include "common.cuh"

// ---------------------------------------------------------------------------------- the walk
// A block owns 32 value columns of one head of one request; eight lanes share a column, each with C consecutive key
// channels of the state in registers (8 C >= dk; channels beyond dk hold zeros). The tokens' vectors are staged in
// shared memory LS_TB at a time. State layout per slot: [head, value channel, key channel].
constexpr int LS_COLS = 32;
constexpr int LS_LANES = 8;
constexpr int LS_TB = 8;
constexpr int LS_THREADS = LS_COLS * LS_LANES;

template <int C>
__global__ void __launch_bounds__(LS_THREADS)
linear_state_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                         const float* __restrict__ w, int ldw, int w_per_channel, const float* __restrict__ bonus,
                         const float* __restrict__ v_scale, float* __restrict__ state, long long state_ld, int state_off,
                         const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ o, int ldo,
                         int heads, int kq_heads, int dk, int dv, float q_scale) {
    constexpr int DKP = LS_LANES * C;
    __shared__ __align__(16) float q_s[LS_TB][DKP];
    __shared__ __align__(16) float k_s[LS_TB][DKP];
    __shared__ __align__(16) float w_s[LS_TB][DKP];
    __shared__ float v_s[LS_TB][LS_COLS];
    const int req = blockIdx.z, h = blockIdx.y;
    const int hq = h / (heads / kq_heads);
    const int lane = threadIdx.x & (LS_LANES - 1), col = threadIdx.x / LS_LANES;
    const int j = blockIdx.x * LS_COLS + col;
    const int row0 = q_start[req], row1 = q_start[req + 1];
    const int c0 = lane * C;
    float* srow = state + (long long)slots[req] * state_ld + state_off + ((long long)h * dv + j) * dk;
    float S[C], U[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
        S[i] = (j < dv && c0 + i < dk) ? srow[c0 + i] : 0.f;
        U[i] = (bonus != nullptr && c0 + i < dk) ? bonus[(size_t)h * dk + c0 + i] : 0.f;
    }
    const bool with_bonus = bonus != nullptr;
    for (int base = row0; base < row1; base += LS_TB) {
        const int nt = min(LS_TB, row1 - base);
        __syncthreads();        // the chunk before has been walked
        for (int e = threadIdx.x; e < LS_TB * DKP; e += LS_THREADS) {
            const int tt = e / DKP, c = e % DKP;
            float qv = 0.f, kv = 0.f, wv = 1.f;
            if (tt < nt && c < dk) {
                const size_t row = (size_t)(base + tt);
                qv = q[row * ldq + (size_t)hq * dk + c] * q_scale;
                kv = k[row * ldk + (size_t)hq * dk + c];
                wv = w_per_channel ? w[row * ldw + (size_t)h * dk + c] : w[row * ldw + h];
            }
            q_s[tt][c] = qv; k_s[tt][c] = kv; w_s[tt][c] = wv;
        }
        for (int e = threadIdx.x; e < LS_TB * LS_COLS; e += LS_THREADS) {
            const int tt = e / LS_COLS, cc = e % LS_COLS, jj = blockIdx.x * LS_COLS + cc;
            float vv = 0.f;
            if (tt < nt && jj < dv) {
                const size_t row = (size_t)(base + tt);
                vv = v[row * ldv + (size_t)h * dv + jj];
                if (v_scale != nullptr) vv *= v_scale[row * heads + h];
            }
            v_s[tt][cc] = vv;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vv = v_s[tt][col];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < C; ++i) {
                const float kv = k_s[tt][c0 + i] * vv;
                if (with_bonus) {
                    acc = fmaf(q_s[tt][c0 + i], fmaf(U[i], kv, S[i]), acc);
                    S[i] = fmaf(w_s[tt][c0 + i], S[i], kv);
                } else {
                    S[i] = fmaf(w_s[tt][c0 + i], S[i], kv);
                    acc = fmaf(q_s[tt][c0 + i], S[i], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (lane == 0 && j < dv) o[(size_t)(base + tt) * ldo + (size_t)h * dv + j] = acc;
        }
    }
    if (j < dv) {
#pragma unroll
        for (int i = 0; i < C; ++i)
            if (c0 + i < dk) srow[c0 + i] = S[i];
    }
}

NIB_API int nib_linear_state_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* w, int ldw,
                                  int w_per_channel, const float* bonus, const float* v_scale, float* state, long long state_ld,
                                  int state_off, const int* q_start, const int* slots, float* o, int ldo, int n_req, int heads,
                                  int kq_heads, int dk, int dv, float q_scale, cudaStream_t stream) {
    NIB_REQUIRE(heads > 0 && kq_heads > 0 && heads % kq_heads == 0, "linear_state_scan: %d heads do not share %d key heads", heads, kq_heads);
    NIB_REQUIRE(dk > 0 && dk <= 256 && dv > 0, "linear_state_scan: key size %d is outside 1..256", dk);
    if (n_req <= 0) return 0;
    const dim3 grid(ceil_div(dv, LS_COLS), heads, n_req), block(LS_THREADS);
#define NIB_LS_LAUNCH(C)                                                                                                     \
    linear_state_scan_kernel<C><<<grid, block, 0, stream>>>(q, ldq, k, ldk, v, ldv, w, ldw, w_per_channel, bonus, v_scale, state, \
                                                            state_ld, state_off, q_start, slots, o, ldo, heads, kq_heads, dk, dv, q_scale)
    if (dk <= 32) NIB_LS_LAUNCH(4);
    else if (dk <= 64) NIB_LS_LAUNCH(8);
    else if (dk <= 128) NIB_LS_LAUNCH(16);
    else NIB_LS_LAUNCH(32);
#undef NIB_LS_LAUNCH
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- short causal convolution
// y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - (taps-1-j), c]) within each request; inputs before the step's first token
// come from the state's history rows (state[slot, off + i * width + c], i = 0 oldest .. taps-2), zeros at a request's
// start. One thread per (token, channel), taps added in ascending order. act: 0 none, 1 silu.
__global__ void __launch_bounds__(256)
conv_tokens_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias, int act,
                   const float* __restrict__ state, long long state_ld, int state_off, const int* __restrict__ q_start,
                   const int* __restrict__ req_index, const int* __restrict__ slots, float* __restrict__ y, int ldy,
                   int tokens, int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)tokens * width) return;
    const int t = (int)(e / width), c = (int)(e % width);
    const int r = req_index[t], first = q_start[r];
    const int i = t - first;
    const float* hist = state != nullptr ? state + (long long)slots[r] * state_ld + state_off : nullptr;
    float acc = bias != nullptr ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int s = i - (taps - 1) + j;
        const float u = s >= 0 ? x[(size_t)(first + s) * ldx + c] : hist[(size_t)(taps - 1 + s) * width + c];
        acc = fmaf(w[(size_t)c * taps + j], u, acc);
    }
    if (act == 1) acc = acc / (1.0f + expf(-acc));
    y[(size_t)t * ldy + c] = acc;
}

// The history rows become the request's last taps-1 inputs (old rows move up when the step brought fewer). One thread
// per (request, channel); row i is written after rows >= i were read, so the move is safe in place.
__global__ void __launch_bounds__(256)
conv_tail_kernel(const float* __restrict__ x, int ldx, float* __restrict__ state, long long state_ld, int state_off,
                 const int* __restrict__ q_start, const int* __restrict__ slots, int n_req, int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)n_req * width) return;
    const int r = (int)(e / width), c = (int)(e % width);
    const int first = q_start[r], len = q_start[r + 1] - first;
    float* hist = state + (long long)slots[r] * state_ld + state_off;
    for (int i = 0; i < taps - 1; ++i) {
        const int s = len - (taps - 1) + i;
        hist[(size_t)i * width + c] = s >= 0 ? x[(size_t)(first + s) * ldx + c] : hist[(size_t)(taps - 1 + s) * width + c];
    }
}

NIB_API int nib_conv_tokens(const float* x, int ldx, const float* w, const float* bias, int act, const float* state, long long state_ld,
                            int state_off, const int* q_start, const int* req_index, const int* slots, float* y, int ldy, int tokens,
                            int width, int taps, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && width > 0 && taps >= 1 && (taps == 1 || state != nullptr), "conv_tokens: bad sizes or no state for %d taps", taps);
    if (tokens == 0) return 0;
    NIB_CUDA(launch_pdl(conv_tokens_kernel, dim3(ceil_div((long long)tokens * width, 256)), dim3(256), (size_t)0, stream, x, ldx, w, bias, act,
                        state, state_ld, state_off, q_start, req_index, slots, y, ldy, tokens, width, taps));
    NIB_LAUNCH_CHECK();
    return 0;
}

NIB_API int nib_conv_tail(const float* x, int ldx, float* state, long long state_ld, int state_off, const int* q_start, const int* slots,
                          int n_req, int width, int taps, cudaStream_t stream) {
    NIB_REQUIRE(n_req >= 0 && width > 0 && taps >= 1, "conv_tail: bad sizes");
    if (n_req == 0 || taps == 1) return 0;
    NIB_CUDA(launch_pdl(conv_tail_kernel, dim3(ceil_div((long long)n_req * width, 256)), dim3(256), (size_t)0, stream, x, ldx, state, state_ld,
                        state_off, q_start, slots, n_req, width, taps));
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- token shift
// out[s, t, :] = h[t] + (h[t-1] - h[t]) * mu[s] for every stream s; h[t-1] of a request's first token in the step is the
// state's row (zeros at the request's start), which then becomes the request's last h. The thread of a request's first
// token reads the state before it writes it; no other thread touches that element.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu, int streams, float* __restrict__ state, long long state_ld,
                   int state_off, const int* __restrict__ q_start, const int* __restrict__ req_index, const int* __restrict__ slots,
                   T* __restrict__ out, int tokens, int width) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)tokens * width) return;
    const int t = (int)(e / width), c = (int)(e % width);
    const int r = req_index[t], first = q_start[r];
    const float cur = Elem<T>::load(h + (size_t)t * width + c);
    float prev;
    if (t > first) {
        prev = Elem<T>::load(h + (size_t)(t - 1) * width + c);
    } else {
        float* st = state + (long long)slots[r] * state_ld + state_off + c;
        prev = *st;
        *st = Elem<T>::load(h + (size_t)(q_start[r + 1] - 1) * width + c);
    }
    const float d = prev - cur;
    for (int s = 0; s < streams; ++s)
        Elem<T>::store(out + ((size_t)s * tokens + t) * width + c, fmaf(d, mu[(size_t)s * width + c], cur));
}

NIB_API int nib_token_shift(const void* h, const float* mu, int streams, float* state, long long state_ld, int state_off,
                            const int* q_start, const int* req_index, const int* slots, void* out, int tokens, int width, int dtype,
                            cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && width > 0 && streams > 0, "token_shift: bad sizes");
    if (tokens == 0) return 0;
    const dim3 grid(ceil_div((long long)tokens * width, 256));
    if (dtype == NIB_F32) NIB_CUDA(launch_pdl(token_shift_kernel<float>, grid, dim3(256), (size_t)0, stream, (const float*)h, mu, streams, state, state_ld, state_off, q_start, req_index, slots, (float*)out, tokens, width));
    else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(token_shift_kernel<__nv_bfloat16>, grid, dim3(256), (size_t)0, stream, (const __nv_bfloat16*)h, mu, streams, state, state_ld, state_off, q_start, req_index, slots, (__nv_bfloat16*)out, tokens, width));
    else NIB_REQUIRE(false, "token_shift: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- decays
// kind 0: sigmoid(z)^(1/param) = exp(log_sigmoid(z) / param); kind 1: exp(-exp(z)). 64-bit inside, rounded once.
__global__ void __launch_bounds__(256)
decay_map_kernel(const float* __restrict__ z, int ldz, float* __restrict__ out, int ldo, int rows, int width, int kind, float param) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)rows * width) return;
    const int t = (int)(e / width), c = (int)(e % width);
    const double x = (double)z[(size_t)t * ldz + c];
    double r;
    if (kind == 0) {
        const double ls = x >= 0.0 ? -log1p(exp(-x)) : x - log1p(exp(x));
        r = exp(ls / (double)param);
    } else {
        r = exp(-exp(x));
    }
    out[(size_t)t * ldo + c] = (float)r;
}

NIB_API int nib_decay_map(const float* z, int ldz, float* out, int ldo, int rows, int width, int kind, float param, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && width > 0 && (kind == 0 || kind == 1) && (kind == 1 || param > 0.f), "decay_map: bad sizes, kind or parameter");
    if (rows == 0) return 0;
    NIB_CUDA(launch_pdl(decay_map_kernel, dim3(ceil_div((long long)rows * width, 256)), dim3(256), (size_t)0, stream, z, ldz, out, ldo, rows, width, kind, param));
    NIB_LAUNCH_CHECK();
    return 0;
}

// dt = softplus(raw + bias[h]) (no clamp), decay = exp(-exp(a_log[h]) * dt), per (token, head).
__global__ void __launch_bounds__(256)
step_sizes_kernel(const float* __restrict__ raw, int ld, const float* __restrict__ bias, const float* __restrict__ a_log,
                  float* __restrict__ dt, float* __restrict__ decay, int tokens, int heads) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)tokens * heads) return;
    const int t = (int)(e / heads), h = (int)(e % heads);
    const double x = (double)(raw[(size_t)t * ld + h] + bias[h]);
    const float step = (float)(x > 0.0 ? x + log1p(exp(-x)) : log1p(exp(x)));
    dt[e] = step;
    decay[e] = (float)exp(-exp((double)a_log[h]) * (double)step);
}

NIB_API int nib_step_sizes(const float* raw, int ld, const float* bias, const float* a_log, float* dt, float* decay, int tokens,
                           int heads, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0, "step_sizes: bad sizes");
    if (tokens == 0) return 0;
    NIB_CUDA(launch_pdl(step_sizes_kernel, dim3(ceil_div((long long)tokens * heads, 256)), dim3(256), (size_t)0, stream, raw, ld, bias, a_log, dt, decay, tokens, heads));
    NIB_LAUNCH_CHECK();
    return 0;
}
