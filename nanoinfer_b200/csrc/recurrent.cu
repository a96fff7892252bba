// Recurrent mixers over a flat batch of requests: each request brings any number of tokens (a prompt's portion or
// one decoded token), its state lives in 32-bit floats in a slot of a state tensor and is carried from step to step.
// Every kernel walks a request's tokens in order with the same arithmetic per token whatever the cut, so a
// position's result does not depend on how the request was cut into steps or on what else is in the batch.
// Which request owns which rows and which slot is read from device arrays (q_start, slots), so a captured graph
// can replay the launches for other requests.
//
//  * generalized delta rule: per head a matrix state S [key channel x value channel];
//      S <- diag(w) S - (a * u)(u^T S) + k v^T   (both products read the old S),   o = S^T r
//    with w = exp(-exp(-1/2) sigmoid(w_logit)), a = sigmoid(a_logit), u = k / sqrt(sum k^2 + 1e-6).
//    The value columns of S are independent of one another: a block owns 16 columns of one head of one request,
//    eight lanes share a column (each holds a slice of the key channels in registers), the token's vectors are
//    staged in shared memory a chunk of tokens at a time.
//  * short causal convolution per channel with its last taps-1 inputs kept in the state;
//  * real-gated linear recurrent unit: S <- a S + sqrt(1 - a^2) (i * u), a = exp(-8 r softplus(lam)), r and i
//    sigmoids of block-diagonal products of u (computed by the matrix kernels before), output S * gelu(y).
#include "common.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------- generalized delta rule
constexpr int DR_CV = 16;      // value columns per block
constexpr int DR_LPC = 8;      // lanes per column
constexpr int DR_THREADS = DR_CV * DR_LPC;

template <int KR>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ a_logit, int ld, const float* __restrict__ w_logit, int ldw,
                       float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ slots,
                       float* __restrict__ o, int ldo, int heads, int d) {
    constexpr int DP = DR_LPC * KR;                 // key channels with padding
    constexpr int TC = DP <= 128 ? 16 : 8;          // tokens staged at a time
    __shared__ float s_w[TC][DP], s_au[TC][DP], s_u[TC][DP], s_k[TC][DP], s_r[TC][DP];
    __shared__ float s_v[TC][DR_CV];
    const int tid = threadIdx.x, lane8 = tid % DR_LPC, col_local = tid / DR_LPC;
    const int head = blockIdx.y, req = blockIdx.z;
    const int col = blockIdx.x * DR_CV + col_local;
    const int t0 = q_start[req], n_tok = q_start[req + 1] - t0;
    const int slot = slots[req];
    const bool col_ok = col < d;
    // state layout: [slot, head, value column, key channel]
    float* st = state + (((size_t)slot * heads + head) * d + (col_ok ? col : 0)) * d;
    float s[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int ch = lane8 * KR + i;
        s[i] = (col_ok && ch < d) ? st[ch] : 0.f;
    }
    const size_t hoff = (size_t)head * d;
    for (int c0 = 0; c0 < n_tok; c0 += TC) {
        const int nc = min(TC, n_tok - c0);
        __syncthreads();       // the chunk before has been read
        for (int idx = tid; idx < TC * DP; idx += DR_THREADS) {
            const int t = idx / DP, ch = idx % DP;
            float kk = 0.f, rr = 0.f, ww = 0.f, aa = 0.f;
            if (t < nc && ch < d) {
                const size_t row = (size_t)(t0 + c0 + t);
                kk = k[row * ld + hoff + ch];
                rr = r[row * ld + hoff + ch];
                aa = sigmoidf_(a_logit[row * ld + hoff + ch]);
                ww = expf(-0.60653065971263342f * sigmoidf_(w_logit[row * ldw + hoff + ch]));
            }
            s_k[t][ch] = kk; s_r[t][ch] = rr; s_w[t][ch] = ww; s_au[t][ch] = aa;
        }
        for (int idx = tid; idx < TC * DR_CV; idx += DR_THREADS) {
            const int t = idx / DR_CV, c = idx % DR_CV;
            const int cc = blockIdx.x * DR_CV + c;
            s_v[t][c] = (t < nc && cc < d) ? v[(size_t)(t0 + c0 + t) * ld + hoff + cc] : 0.f;
        }
        __syncthreads();
        // the unit key: one warp per token, lanes over the channels, a fixed order of additions
        for (int t = tid >> 5; t < nc; t += DR_THREADS / 32) {
            float ss = 0.f;
            for (int ch = tid & 31; ch < DP; ch += 32) ss = fmaf(s_k[t][ch], s_k[t][ch], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss + 1e-6f);
            for (int ch = tid & 31; ch < DP; ch += 32) {
                const float u = s_k[t][ch] * inv;
                s_u[t][ch] = u;
                s_au[t][ch] *= u;
            }
        }
        __syncthreads();
        for (int t = 0; t < nc; ++t) {
            const float* pu = &s_u[t][lane8 * KR];
            const float* pw = &s_w[t][lane8 * KR];
            const float* pa = &s_au[t][lane8 * KR];
            const float* pk = &s_k[t][lane8 * KR];
            const float* pr = &s_r[t][lane8 * KR];
            float proj = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) proj = fmaf(pu[i], s[i], proj);
            proj += __shfl_xor_sync(0xffffffffu, proj, 1);
            proj += __shfl_xor_sync(0xffffffffu, proj, 2);
            proj += __shfl_xor_sync(0xffffffffu, proj, 4);
            const float vj = s_v[t][col_local];
            float out = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                s[i] = fmaf(pk[i], vj, fmaf(-pa[i], proj, pw[i] * s[i]));
                out = fmaf(s[i], pr[i], out);
            }
            out += __shfl_xor_sync(0xffffffffu, out, 1);
            out += __shfl_xor_sync(0xffffffffu, out, 2);
            out += __shfl_xor_sync(0xffffffffu, out, 4);
            if (lane8 == 0 && col_ok) o[(size_t)(t0 + c0 + t) * ldo + hoff + col] = out;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            const int ch = lane8 * KR + i;
            if (ch < d) st[ch] = s[i];
        }
    }
}

// r, k, v, a_logit: [tokens, heads*d] floats with row stride ld; w_logit likewise with row stride ldw;
// state: [slots, heads, d, d] floats; o: [tokens, heads*d] floats with row stride ldo.
NIB_API int nib_delta_rule_scan(const float* r, const float* k, const float* v, const float* a_logit, int ld,
                                const float* w_logit, int ldw, float* state, const int* q_start, const int* slots,
                                float* o, int ldo, int requests, int heads, int d, cudaStream_t stream) {
    NIB_REQUIRE(requests >= 0 && heads > 0 && d > 0 && d <= 256, "delta_rule_scan: head size %d is outside 1..256", d);
    if (requests == 0) return 0;
    const dim3 grid(ceil_div(d, DR_CV), heads, requests);
    const int kr = ceil_div(d, DR_LPC);
#define NIB_DR(KR)                                                                                                      \
    if (kr <= KR) {                                                                                                     \
        delta_rule_scan_kernel<KR><<<grid, DR_THREADS, 0, stream>>>(r, k, v, a_logit, ld, w_logit, ldw, state, q_start, \
                                                                    slots, o, ldo, heads, d);                          \
        NIB_LAUNCH_CHECK();                                                                                             \
        return 0;                                                                                                       \
    }
    NIB_DR(1) NIB_DR(2) NIB_DR(3) NIB_DR(4) NIB_DR(6) NIB_DR(8) NIB_DR(12) NIB_DR(16) NIB_DR(24) NIB_DR(32)
#undef NIB_DR
    NIB_REQUIRE(false, "delta_rule_scan: head size %d", d);
    return 0;
}

// ---------------------------------------------------------------------------------- short causal convolution
// u[t, c] = bias[c] + sum_j w[c, j] * x[t - (taps-1-j), c] over the request's own positions; inputs before this
// step's first token come from the state's history rows (the last taps-1 inputs of earlier steps, zeros at the
// start of a request). Writes u in 32-bit [tokens, width] and, for the block-diagonal products that follow, in the
// storage type laid out block by block: [blocks, tokens, width / blocks].
// state: [slots, rows_per_slot, width]; history rows are rows hist_row0 .. hist_row0 + taps - 2 (oldest first).
template <typename T>
__global__ void causal_conv_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, int rows_per_slot, int hist_row0,
                                   const int* __restrict__ q_start, const int* __restrict__ req_index, const int* __restrict__ slots,
                                   float* __restrict__ u32, T* __restrict__ u_blocks, int tokens, int width, int taps, int blocks) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    const int req = req_index[t];
    const int local = t - q_start[req];
    const float* hist = state + ((size_t)slots[req] * rows_per_slot + hist_row0) * width;
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {
        const int src = local - (taps - 1 - j);
        const float xv = src >= 0 ? x[(size_t)(t - (taps - 1 - j)) * ldx + c] : hist[(size_t)(local + j) * width + c];
        acc = fmaf(w[(size_t)c * taps + j], xv, acc);
    }
    u32[(size_t)t * width + c] = acc;
    const int bw = width / blocks;
    Elem<T>::store(u_blocks + ((size_t)(c / bw) * tokens + t) * bw + (c % bw), acc);
}

NIB_API int nib_causal_conv(const float* x, int ldx, const float* w, const float* bias, const float* state, int rows_per_slot,
                            int hist_row0, const int* q_start, const int* req_index, const int* slots, float* u32,
                            void* u_blocks, int tokens, int width, int taps, int blocks, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && width > 0 && taps >= 1 && blocks >= 1 && width % blocks == 0, "causal_conv: bad sizes");
    if (tokens == 0) return 0;
    const int grid = ceil_div((long long)tokens * width, 256);
    if (dtype == NIB_F32)
        causal_conv_kernel<float><<<grid, 256, 0, stream>>>(x, ldx, w, bias, state, rows_per_slot, hist_row0, q_start, req_index,
                                                            slots, u32, (float*)u_blocks, tokens, width, taps, blocks);
    else if (dtype == NIB_BF16)
        causal_conv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(x, ldx, w, bias, state, rows_per_slot, hist_row0, q_start,
                                                                    req_index, slots, u32, (__nv_bfloat16*)u_blocks, tokens, width, taps, blocks);
    else
        NIB_REQUIRE(false, "causal_conv: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- gated linear recurrence
// One thread per (request, channel) walks the request's tokens. gates: [blocks, tokens, 2 * bw] floats, the
// recurrence gate's logits in the first bw columns of a block's rows and the input gate's in the last bw.
// y_logit: the other branch before its gelu, row stride ldy. x: the convolution's inputs (row stride ldx), from
// which the history rows of the state are renewed. state row 0 is S, rows 1.. the history.
constexpr int LRU_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float* __restrict__ u32, const float* __restrict__ gates, const float* __restrict__ y_logit, int ldy,
                  const float* __restrict__ x, int ldx, const float* __restrict__ softplus_lam, float* __restrict__ state,
                  const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ out, int tokens, int width,
                  int taps, int blocks) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int req = blockIdx.y;
    const int t0 = q_start[req], n = q_start[req + 1] - t0;
    float* st = state + (size_t)slots[req] * taps * width;
    const int bw = width / blocks, b = c / bw, cb = c % bw;
    const float* g = gates + ((size_t)b * tokens) * 2 * bw + cb;
    const float sp = softplus_lam[c];
    float S = st[c];
#pragma unroll 4
    for (int t = 0; t < n; ++t) {
        const size_t row = (size_t)(t0 + t);
        const float rg = sigmoidf_(g[row * 2 * bw]), ig = sigmoidf_(g[row * 2 * bw + bw]);
        const float log_a = -8.0f * rg * sp;
        const float a = expf(log_a);
        const float mult = sqrtf(fmaxf(0.f, -expm1f(2.0f * log_a)));      // sqrt(1 - a^2)
        S = fmaf(a, S, mult * (ig * u32[row * width + c]));
        const float z = y_logit[row * ldy + c];
        const float ge = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        Elem<T>::store(out + row * width + c, S * ge);
    }
    st[c] = S;
    // the last taps-1 inputs: from this step's rows where there are enough, else shifted up from the old history
    float keep[LRU_MAX_TAPS];
    for (int j = 0; j < taps - 1; ++j) {
        const int src = n - (taps - 1) + j;
        keep[j] = src >= 0 ? x[(size_t)(t0 + src) * ldx + c] : st[(size_t)(1 + j + n) * width + c];
    }
    for (int j = 0; j < taps - 1; ++j) st[(size_t)(1 + j) * width + c] = keep[j];
}

NIB_API int nib_rglru_scan(const float* u32, const float* gates, const float* y_logit, int ldy, const float* x, int ldx,
                           const float* softplus_lam, float* state, const int* q_start, const int* slots, void* out,
                           int tokens, int requests, int width, int taps, int blocks, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(requests >= 0 && width > 0 && taps >= 1 && taps <= LRU_MAX_TAPS && blocks >= 1 && width % blocks == 0,
                "rglru_scan: bad sizes (width %d, taps %d of at most %d, blocks %d)", width, taps, LRU_MAX_TAPS, blocks);
    if (requests == 0 || tokens == 0) return 0;
    const dim3 grid(ceil_div(width, 128), requests);
    if (dtype == NIB_F32)
        rglru_scan_kernel<float><<<grid, 128, 0, stream>>>(u32, gates, y_logit, ldy, x, ldx, softplus_lam, state, q_start, slots,
                                                           (float*)out, tokens, width, taps, blocks);
    else if (dtype == NIB_BF16)
        rglru_scan_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(u32, gates, y_logit, ldy, x, ldx, softplus_lam, state, q_start,
                                                                   slots, (__nv_bfloat16*)out, tokens, width, taps, blocks);
    else
        NIB_REQUIRE(false, "rglru_scan: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}
