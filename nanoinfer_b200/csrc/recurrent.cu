// Recurrent mixers over a flat batch of requests: each request brings any number of tokens (a prompt's portion or
// one decoded token), its state lives in 32-bit floats in a slot of a state tensor and is carried from step to step.
// The delta rule and the convolution walk a request's tokens in order with the same arithmetic per token whatever
// the cut; the gated recurrence chains segments of the request's tokens, so its results depend on the cut by
// rounding only. Nothing depends on what else is in the batch.
// Which request owns which rows and which slot is read from device arrays (q_start, slots), so a captured graph
// can replay the launches for other requests.
//
//  * generalized delta rule: per head a matrix state S [key channel x value channel];
//      S <- diag(w) S - (a * u)(u^T S) + k v^T   (both products read the old S),   o = S^T r
//    with w = exp(-exp(-1/2) sigmoid(w_logit)), a = sigmoid(a_logit), u = k / sqrt(sum k^2 + 1e-6).
//    Decay, unit key and removal are computed for all tokens in parallel first. The value columns of S are
//    independent of one another: a block owns 16 columns of one head of one request, eight lanes share a column
//    (each holds a slice of the key channels in registers), the tokens' vectors are staged in shared memory a chunk
//    at a time; what a token costs is the chain projection -> butterfly over the eight lanes -> update.
//  * short causal convolution per channel with its last taps-1 inputs kept in the state;
//  * real-gated linear recurrent unit: S <- a S + sqrt(1 - a^2) (i * u), a = exp(-8 r softplus(lam)), r and i
//    sigmoids of block-diagonal products of u (computed by the matrix kernels before), output S * gelu(y).
#include "common.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------- generalized delta rule
// Two kernels. The first is parallel over (token, head), a warp each: decay w, unit key u and a * u from the logits
// and the key, into work[0], work[1], work[2] ([3, tokens, heads*d] floats). The second walks the tokens.
constexpr int DR_CV = 16;      // value columns per block
constexpr int DR_LPC = 8;      // lanes per column
constexpr int DR_THREADS = DR_CV * DR_LPC;

__global__ void __launch_bounds__(128)
delta_rule_prepare_kernel(const float* __restrict__ k, const float* __restrict__ a_logit, int ld, const float* __restrict__ w_logit,
                          int ldw, float* __restrict__ work, int tokens, int heads, int d) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)tokens * heads) return;
    const int t = (int)(wid / heads), h = (int)(wid % heads);
    const size_t in = (size_t)t * ld + (size_t)h * d, inw = (size_t)t * ldw + (size_t)h * d;
    const size_t plane = (size_t)tokens * heads * d, out = ((size_t)t * heads + h) * d;
    float ss = 0.f;
    for (int ch = lane; ch < d; ch += 32) ss = fmaf(k[in + ch], k[in + ch], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
    for (int ch = lane; ch < d; ch += 32) {
        const float u = k[in + ch] * inv;
        // exp(-exp(-1/2) sigmoid), rounded to 32 bits once from a 64-bit exponential (see rglru_gate_kernel)
        work[out + ch] = (float)exp(-0.60653065971263342 * (double)sigmoidf_(w_logit[inw + ch]));
        work[plane + out + ch] = u;
        work[2 * plane + out + ch] = sigmoidf_(a_logit[in + ch]) * u;
    }
}

template <int KR>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v, int ld,
                       const float* __restrict__ work, float* __restrict__ state, const int* __restrict__ q_start,
                       const int* __restrict__ slots, float* __restrict__ o, int ldo, int tokens, int heads, int d) {
        pdl_wait();      // everything this kernel reads may come from the kernel before
    constexpr bool VEC = KR % 4 == 0;
    // a lane's slice, padded to an odd number of 16-byte units so that the eight lanes' 16-byte loads fall into distinct banks
    constexpr int KRP = (VEC && (KR / 4) % 2 == 0) ? KR + 4 : KR;
    constexpr int DP = DR_LPC * KR;                 // key channels with padding
    constexpr int DPP = DR_LPC * KRP;
    constexpr int TC = DPP <= 96 ? 16 : 8;          // tokens staged at a time
    __shared__ __align__(16) float s_w[TC][DPP], s_au[TC][DPP], s_u[TC][DPP], s_k[TC][DPP], s_r[TC][DPP];
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
    const size_t hoff = (size_t)head * d, n_all = (size_t)heads * d, plane = (size_t)tokens * n_all;
    // A chunk's vectors are fetched into registers while the chunk before is being walked: the walk never waits
    // for global memory.
    constexpr int PER = (TC * DP + DR_THREADS - 1) / DR_THREADS;        // (token, channel) pairs per thread
    constexpr int PERV = (TC * DR_CV + DR_THREADS - 1) / DR_THREADS;
    float f_k[PER], f_r[PER], f_a[PER], f_w[PER], f_u[PER], f_v[PERV];
    auto fetch = [&](int c0) {
        const int nc = min(TC, n_tok - c0);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = tid + j * DR_THREADS, t = idx / DP, ch = idx % DP;
            f_k[j] = f_r[j] = f_a[j] = f_w[j] = f_u[j] = 0.f;
            if (idx < TC * DP && t < nc && ch < d) {
                const size_t row = (size_t)(t0 + c0 + t);
                f_k[j] = k[row * ld + hoff + ch];
                f_r[j] = r[row * ld + hoff + ch];
                f_w[j] = work[row * n_all + hoff + ch];
                f_u[j] = work[plane + row * n_all + hoff + ch];
                f_a[j] = work[2 * plane + row * n_all + hoff + ch];
            }
        }
#pragma unroll
        for (int j = 0; j < PERV; ++j) {
            const int idx = tid + j * DR_THREADS, t = idx / DR_CV, cc = blockIdx.x * DR_CV + idx % DR_CV;
            f_v[j] = (idx < TC * DR_CV && t < nc && cc < d) ? v[(size_t)(t0 + c0 + t) * ld + hoff + cc] : 0.f;
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = tid + j * DR_THREADS, t = idx / DP, ch = idx % DP;
            if (idx >= TC * DP) continue;
            const int at = (ch / KR) * KRP + ch % KR;
            s_k[t][at] = f_k[j]; s_r[t][at] = f_r[j]; s_w[t][at] = f_w[j]; s_u[t][at] = f_u[j]; s_au[t][at] = f_a[j];
        }
#pragma unroll
        for (int j = 0; j < PERV; ++j) {
            const int idx = tid + j * DR_THREADS;
            if (idx < TC * DR_CV) s_v[idx / DR_CV][idx % DR_CV] = f_v[j];
        }
        __syncthreads();
    };
    auto take = [&](float (&dst)[KR], const float* src) {
        if constexpr (VEC) {
#pragma unroll
            for (int i = 0; i < KR / 4; ++i) {
                const float4 x = reinterpret_cast<const float4*>(src)[i];
                dst[4 * i] = x.x; dst[4 * i + 1] = x.y; dst[4 * i + 2] = x.z; dst[4 * i + 3] = x.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < KR; ++i) dst[i] = src[i];
        }
    };
    if (n_tok > 0) fetch(0);
    float out_prev = 0.f;       // the token before's output, summed over the lanes while this token's projection is
    long long prev_at = -1;
    for (int c0 = 0; c0 < n_tok; c0 += TC) {
        const int nc = min(TC, n_tok - c0);
        __syncthreads();       // the chunk before has been walked
        stage();
        if (c0 + TC < n_tok) fetch(c0 + TC);
        for (int t = 0; t < nc; ++t) {
            float cu[KR], cw[KR], ca[KR], ck[KR], cr[KR];
            take(cu, &s_u[t][lane8 * KRP]);
            take(cw, &s_w[t][lane8 * KRP]);
            take(ca, &s_au[t][lane8 * KRP]);
            take(ck, &s_k[t][lane8 * KRP]);
            take(cr, &s_r[t][lane8 * KRP]);
            const float vj = s_v[t][col_local];
            float p0 = 0.f, p1 = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                if (i & 1) p1 = fmaf(cu[i], s[i], p1); else p0 = fmaf(cu[i], s[i], p0);
            }
            float proj = p0 + p1;
#pragma unroll
            for (int m = 1; m < DR_LPC; m <<= 1) {      // two independent butterflies side by side
                const float x = __shfl_xor_sync(0xffffffffu, proj, m), y = __shfl_xor_sync(0xffffffffu, out_prev, m);
                proj += x; out_prev += y;
            }
            if (prev_at >= 0 && lane8 == 0 && col_ok) o[prev_at] = out_prev;
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                s[i] = fmaf(ck[i], vj, fmaf(-ca[i], proj, cw[i] * s[i]));
                if (i & 1) o1 = fmaf(s[i], cr[i], o1); else o0 = fmaf(s[i], cr[i], o0);
            }
            out_prev = o0 + o1;
            prev_at = (long long)(t0 + c0 + t) * ldo + hoff + col;
        }
    }
    pdl_launch_dependents();        // only now: blocks of the next kernel that became resident earlier would sit beside a long walk
    if (prev_at >= 0) {
#pragma unroll
        for (int m = 1; m < DR_LPC; m <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, m);
        if (lane8 == 0 && col_ok) o[prev_at] = out_prev;
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
// state: [slots, heads, d, d] floats; o: [tokens, heads*d] floats with row stride ldo; work: [3, tokens, heads*d]
// floats of scratch.
NIB_API int nib_delta_rule_scan(const float* r, const float* k, const float* v, const float* a_logit, int ld,
                                const float* w_logit, int ldw, float* state, const int* q_start, const int* slots,
                                float* o, int ldo, float* work, int tokens, int requests, int heads, int d, cudaStream_t stream) {
    NIB_REQUIRE(requests >= 0 && heads > 0 && d > 0 && d <= 256, "delta_rule_scan: head size %d is outside 1..256", d);
    if (requests == 0 || tokens == 0) return 0;
    NIB_CUDA(launch_pdl(delta_rule_prepare_kernel, dim3(ceil_div((long long)tokens * heads, 4)), dim3(128), (size_t)(0), stream, k, a_logit, ld, w_logit, ldw, work, tokens, heads, d));
    NIB_LAUNCH_CHECK();
    // The walk is launched plainly, after the kernel before has ended: as a programmatic dependent its few blocks become
    // resident while that kernel still runs, wherever room is first, several to an SM, and the walk of 2,048 tokens took
    // 1.05 ms instead of 0.45 ms (heads of 64).
    const dim3 grid(ceil_div(d, DR_CV), heads, requests);
    const int kr = ceil_div(d, DR_LPC);
#define NIB_DR(KR)                                                                                                         \
    if (kr <= KR) {                                                                                                        \
        delta_rule_scan_kernel<KR><<<grid, DR_THREADS, 0, stream>>>(r, k, v, ld, work, state, q_start, slots, o, ldo, tokens, \
                                                                    heads, d);                                             \
        NIB_LAUNCH_CHECK();                                                                                                \
        return 0;                                                                                                          \
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
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;       // a token per block row: no division per element
    if (c >= width) return;
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
    const dim3 grid(tokens, ceil_div(width, 256));
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(causal_conv_kernel<float>, dim3(grid), dim3(256), (size_t)(0), stream, x, ldx, w, bias, state, rows_per_slot, hist_row0, q_start, req_index,
                                                            slots, u32, (float*)u_blocks, tokens, width, taps, blocks));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(causal_conv_kernel<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)(0), stream, x, ldx, w, bias, state, rows_per_slot, hist_row0, q_start,
                                                                    req_index, slots, u32, (__nv_bfloat16*)u_blocks, tokens, width, taps, blocks));
    else
        NIB_REQUIRE(false, "causal_conv: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- gated linear recurrence
// Two kernels. The first is element-wise over (token, channel): from the gate logits (gates: [blocks, tokens,
// 2 * bw] floats, the recurrence gate's logits in the first bw columns of a block's rows and the input gate's in the
// last bw), u and the other branch's logits it writes a = exp(-8 r softplus(lam)), b = sqrt(1 - a^2) (i u) and
// g = gelu_tanh(y) into work[0], work[1], work[2] ([3, tokens, width] floats). The second walks S <- a S + b:
// a block owns 32 channels of one request (a lane per channel), its warps take consecutive segments of the
// request's tokens; each warp first composes its segment into (product of a, end state from zero), the segments
// are chained in order from the request's state, then each warp walks its segment again from its true entry state
// and writes S * g. Loads are issued eight tokens ahead. State row 0 is S, rows 1.. the last taps-1 inputs x of the
// convolution (row stride ldx), renewed here.
constexpr int LRU_MAX_TAPS = 16;
constexpr int LRU_WARPS = 32;
constexpr int LRU_AHEAD = 8;

__global__ void rglru_gate_kernel(const float* __restrict__ u32, const float* __restrict__ gates, const float* __restrict__ y_logit,
                                  int ldy, const float* __restrict__ softplus_lam, float* __restrict__ work, int tokens, int width,
                                  int blocks) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;       // a token per block row: no division per element
    if (c >= width) return;
    const size_t n = (size_t)tokens * width, i = (size_t)t * width + c;
    const int bw = width / blocks, b = c / bw, cb = c % bw;
    const float* g = gates + ((size_t)b * tokens + t) * 2 * bw + cb;
    const float rg = sigmoidf_(g[0]), ig = sigmoidf_(g[bw]);
    const float log_a = -8.0f * rg * softplus_lam[c];
    // The decay is raised to hundreds of powers along a sequence: it is rounded to 32 bits once, from a 64-bit
    // exponential (expf alone may be two units in the last place off, which a long memory multiplies up).
    const double la = (double)log_a;
    work[i] = (float)exp(la);
    work[n + i] = (float)sqrt(fmax(0.0, -expm1(2.0 * la))) * (ig * u32[i]);      // sqrt(1 - a^2) (i u)
    const float z = y_logit[(size_t)t * ldy + c];
    work[2 * n + i] = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(LRU_WARPS * 32)
rglru_scan_kernel(const float* __restrict__ work, const float* __restrict__ x, int ldx, float* __restrict__ state,
                  const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ out, int tokens, int width, int taps) {
        pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float s_a[LRU_WARPS][32], s_b[LRU_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const bool live = c < width;
    const int req = blockIdx.y;
    const int t0 = q_start[req], n = q_start[req + 1] - t0;
    float* st = state + (size_t)slots[req] * taps * width;
    const size_t plane = (size_t)tokens * width;
    const float* pa = work + (size_t)t0 * width + c;
    const float* pb = pa + plane;
    const float* pg = pb + plane;
    const int seg = (n + LRU_WARPS - 1) / LRU_WARPS;
    const int lo = min(n, warp * seg), hi = min(n, lo + seg);
    // pass 1: the segment as one affine map S -> A S + B
    float A = 1.f, B = 0.f;
    if (live) {
        for (int t = lo; t < hi; t += LRU_AHEAD) {
            float av[LRU_AHEAD], bv[LRU_AHEAD];
#pragma unroll
            for (int j = 0; j < LRU_AHEAD; ++j) {
                const bool in = t + j < hi;
                av[j] = in ? pa[(size_t)(t + j) * width] : 1.f;
                bv[j] = in ? pb[(size_t)(t + j) * width] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < LRU_AHEAD; ++j) { B = fmaf(av[j], B, bv[j]); A *= av[j]; }
        }
    }
    s_a[warp][lane] = A; s_b[warp][lane] = B;
    __syncthreads();
    if (!live) return;
    float S = st[c];
    for (int w = 0; w < warp; ++w) S = fmaf(s_a[w][lane], S, s_b[w][lane]);
    // pass 2: the segment again from its entry state
    for (int t = lo; t < hi; t += LRU_AHEAD) {
        float av[LRU_AHEAD], bv[LRU_AHEAD], gv[LRU_AHEAD];
#pragma unroll
        for (int j = 0; j < LRU_AHEAD; ++j) {
            const bool in = t + j < hi;
            av[j] = in ? pa[(size_t)(t + j) * width] : 1.f;
            bv[j] = in ? pb[(size_t)(t + j) * width] : 0.f;
            gv[j] = in ? pg[(size_t)(t + j) * width] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < LRU_AHEAD; ++j) {
            S = fmaf(av[j], S, bv[j]);
            if (t + j < hi) Elem<T>::store(out + (size_t)(t0 + t + j) * width + c, S * gv[j]);
        }
    }
    pdl_launch_dependents();        // only now: the next kernel's blocks would sit beside the walk
    if (warp != LRU_WARPS - 1) return;
    // the last warp leaves with the request's new state (empty segments are the identity map)
    st[c] = S;
    float keep[LRU_MAX_TAPS];
    for (int j = 0; j < taps - 1; ++j) {
        const int src = n - (taps - 1) + j;
        keep[j] = src >= 0 ? x[(size_t)(t0 + src) * ldx + c] : st[(size_t)(1 + j + n) * width + c];
    }
    for (int j = 0; j < taps - 1; ++j) st[(size_t)(1 + j) * width + c] = keep[j];
}

// A handful of tokens (a decode step): gates, decay and walk in one kernel, one thread per (request, channel).
template <typename T>
__global__ void __launch_bounds__(128)
rglru_few_tokens_kernel(const float* __restrict__ u32, const float* __restrict__ gates, const float* __restrict__ y_logit, int ldy,
                        const float* __restrict__ x, int ldx, const float* __restrict__ softplus_lam, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ out, int tokens, int width,
                        int taps, int blocks) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int req = blockIdx.y;
    const int t0 = q_start[req], n = q_start[req + 1] - t0;
    float* st = state + (size_t)slots[req] * taps * width;
    const int bw = width / blocks, b = c / bw, cb = c % bw;
    const float* g = gates + ((size_t)b * tokens) * 2 * bw + cb;
    const float sp = softplus_lam[c];
    float S = st[c];
    for (int t = 0; t < n; ++t) {
        const size_t row = (size_t)(t0 + t);
        const float rg = sigmoidf_(g[row * 2 * bw]), ig = sigmoidf_(g[row * 2 * bw + bw]);
        const double la = (double)(-8.0f * rg * sp);        // as in rglru_gate_kernel
        S = fmaf((float)exp(la), S, (float)sqrt(fmax(0.0, -expm1(2.0 * la))) * (ig * u32[row * width + c]));
        const float z = y_logit[row * ldy + c];
        Elem<T>::store(out + row * width + c, S * (0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)))));
    }
    st[c] = S;
    float keep[LRU_MAX_TAPS];
    for (int j = 0; j < taps - 1; ++j) {
        const int src = n - (taps - 1) + j;
        keep[j] = src >= 0 ? x[(size_t)(t0 + src) * ldx + c] : st[(size_t)(1 + j + n) * width + c];
    }
    for (int j = 0; j < taps - 1; ++j) st[(size_t)(1 + j) * width + c] = keep[j];
}

// work: [3, tokens, width] floats of scratch.
NIB_API int nib_rglru_scan(const float* u32, const float* gates, const float* y_logit, int ldy, const float* x, int ldx,
                           const float* softplus_lam, float* state, const int* q_start, const int* slots, void* out, float* work,
                           int tokens, int requests, int width, int taps, int blocks, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(requests >= 0 && width > 0 && taps >= 1 && taps <= LRU_MAX_TAPS && blocks >= 1 && width % blocks == 0,
                "rglru_scan: bad sizes (width %d, taps %d of at most %d, blocks %d)", width, taps, LRU_MAX_TAPS, blocks);
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "rglru_scan: unknown dtype %d", dtype);
    if (requests == 0 || tokens == 0) return 0;
    if (tokens <= 16) {         // which kernel runs depends on the step's size alone
        const dim3 few(ceil_div(width, 128), requests);
        if (dtype == NIB_F32)
            NIB_CUDA(launch_pdl(rglru_few_tokens_kernel<float>, few, dim3(128), (size_t)0, stream, u32, gates, y_logit, ldy, x, ldx,
                                softplus_lam, state, q_start, slots, (float*)out, tokens, width, taps, blocks));
        else
            NIB_CUDA(launch_pdl(rglru_few_tokens_kernel<__nv_bfloat16>, few, dim3(128), (size_t)0, stream, u32, gates, y_logit, ldy, x,
                                ldx, softplus_lam, state, q_start, slots, (__nv_bfloat16*)out, tokens, width, taps, blocks));
        return 0;
    }
    NIB_CUDA(launch_pdl(rglru_gate_kernel, dim3(tokens, ceil_div(width, 256)), dim3(256), (size_t)(0), stream, u32, gates, y_logit, ldy, softplus_lam, work,
                                                                                    tokens, width, blocks));
    NIB_LAUNCH_CHECK();
    const dim3 grid(ceil_div(width, 32), requests);
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(rglru_scan_kernel<float>, dim3(grid), dim3(LRU_WARPS * 32), (size_t)(0), stream, work, x, ldx, state, q_start, slots, (float*)out, tokens, width, taps));
    else
        NIB_CUDA(launch_pdl(rglru_scan_kernel<__nv_bfloat16>, dim3(grid), dim3(LRU_WARPS * 32), (size_t)(0), stream, work, x, ldx, state, q_start, slots, (__nv_bfloat16*)out,
                                                                              tokens, width, taps));
    NIB_LAUNCH_CHECK();
    return 0;
}
