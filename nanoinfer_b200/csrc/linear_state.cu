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
// A block owns 16 value columns of one head of one request; eight lanes share a column, each with C key channels of the
// state in registers (8 C >= dk; channels beyond dk hold zeros): lane l owns the channels (8 i + l) * 4 .. + 3, so the
// eight lanes read 128 consecutive bytes of a token's vector with one 16-byte load each. The tokens' vectors are staged
// in shared memory TB at a time by cp.async, three chunks ahead of the one that is walked (rows and columns that do not
// exist arrive as zeros, under which a state element stays zero). What a token costs is 3 C multiply-adds per thread
// and a share of a butterfly over the eight lanes. State layout per slot: [head, value channel, key channel].
constexpr int LS_COLS = 16;
constexpr int LS_LANES = 8;
constexpr int LS_THREADS = LS_COLS * LS_LANES;

__device__ __forceinline__ void ls_cp_async_4(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 4 : 0;    // 0 source bytes: the destination is zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}

// One staged chunk in shared memory: TB tokens' q and k (DKP floats each), decays (DKP, or one per token), the block's
// value columns and the factor on the values. STAGES chunks are in flight: a chunk's loads have the walk of the
// STAGES - 1 chunks before it to arrive.
__device__ __forceinline__ void ls_cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}

template <int C, bool PER_CHANNEL> struct LsLayout {
    static constexpr int DKP = LS_LANES * C;
    static constexpr int TB = 8;                        // as many tokens as lanes share a column: see the butterfly below
    static constexpr int STAGES = C >= 32 ? 2 : 4;
    static constexpr int WP = PER_CHANNEL ? DKP : 4;
    static constexpr int K0 = TB * DKP, W0 = 2 * TB * DKP, V0 = W0 + TB * WP, F0 = V0 + TB * LS_COLS;
    static constexpr int STAGE = F0 + ((TB + 3) / 4) * 4;
    static constexpr int BYTES = STAGES * STAGE * 4;
};

// MODE 0: a request's tokens from its slot's state to its slot's state. For long prompts the tokens are cut into
// segments of seg_len that run side by side: MODE 1 walks every segment but a request's last from a zero state (no
// outputs) and leaves its end state and the product of its decays; ls_combine_kernel chains them into every segment's
// true entry state; MODE 2 walks every segment again from that state with outputs, the last one into the slot.
// seg_state: [request, segment, head, value channel, key channel]; seg_decay: [request, segment, head, key channel or 1].
template <int C, bool PER_CHANNEL, bool BONUS, int MODE>
__global__ void __launch_bounds__(LS_THREADS)
linear_state_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                         const float* __restrict__ w, int ldw, const float* __restrict__ bonus,
                         const float* __restrict__ v_scale, float* __restrict__ state, long long state_ld, int state_off,
                         const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ o, int ldo,
                         int heads, int kq_heads, int dk, int dv, float q_scale, int n_seg, int seg_len,
                         float* __restrict__ seg_state, float* __restrict__ seg_decay, int vec) {
    using L = LsLayout<C, PER_CHANNEL>;
    constexpr int DKP = L::DKP, TB = L::TB, STAGES = L::STAGES;
    extern __shared__ __align__(16) float ls_smem[];
    auto q_s = [&](int buf, int tt) { return ls_smem + buf * L::STAGE + tt * DKP; };
    auto k_s = [&](int buf, int tt) { return ls_smem + buf * L::STAGE + L::K0 + tt * DKP; };
    auto w_s = [&](int buf, int tt) { return ls_smem + buf * L::STAGE + L::W0 + tt * L::WP; };
    auto v_s = [&](int buf, int tt) { return ls_smem + buf * L::STAGE + L::V0 + tt * LS_COLS; };
    auto f_s = [&](int buf) { return ls_smem + buf * L::STAGE + L::F0; };
    const int req = MODE == 0 ? blockIdx.z : blockIdx.z / n_seg, seg = MODE == 0 ? 0 : blockIdx.z % n_seg, h = blockIdx.y;
    const int hq = h / (heads / kq_heads);
    const int lane = threadIdx.x & (LS_LANES - 1), col = threadIdx.x / LS_LANES;
    const int j = blockIdx.x * LS_COLS + col;
    const int req_row1 = q_start[req + 1];
    const int row0 = q_start[req] + (MODE == 0 ? 0 : seg * seg_len);
    const int row1 = MODE == 0 ? req_row1 : min(req_row1, row0 + seg_len);
    if (row0 >= req_row1) return;                       // the request has fewer segments
    const bool last = row1 == req_row1;
    if (MODE == 1 && last) return;                      // a request's last segment ends in the slot, in the second walk
    float* srow = state + (long long)slots[req] * state_ld + state_off + ((long long)h * dv + j) * dk;
    const size_t elems = (size_t)heads * dv * dk;
    float* seg_row = MODE == 0 ? nullptr : seg_state + ((size_t)req * n_seg + seg) * elems + ((size_t)h * dv + j) * dk;
    const bool track = MODE == 1 && blockIdx.x == 0 && col == 0;       // these eight lanes also multiply the segment's decays up
    float S[C], U[C], P[MODE == 1 ? C : 1];
#pragma unroll
    for (int i = 0; i < C; ++i) {
        const int c = ((i >> 2) * LS_LANES + lane) * 4 + (i & 3);
        const float* from = MODE == 2 ? seg_row : srow;
        S[i] = (MODE != 1 && j < dv && c < dk) ? from[c] : 0.f;
        U[i] = (BONUS && c < dk) ? bonus[(size_t)h * dk + c] : 0.f;
        if (MODE == 1) P[i] = 1.f;
    }
    const bool scaled = v_scale != nullptr;

    auto stage = [&](int buf, int base) {
        const int nt = min(TB, row1 - base);
        if (vec) {      // rows of q, k and decays start on 16-byte boundaries and dk is a multiple of 4: four floats a copy
            for (int e = threadIdx.x; e < TB * (DKP / 4); e += LS_THREADS) {
                const int tt = e / (DKP / 4), c = (e % (DKP / 4)) * 4;
                const bool ok = tt < nt && c < dk;
                const size_t row = (size_t)(base + (ok ? tt : 0));
                const int cc = ok ? c : 0;
                if (MODE != 1) ls_cp_async_16(q_s(buf, tt) + c, q + row * ldq + (size_t)hq * dk + cc, ok);
                ls_cp_async_16(k_s(buf, tt) + c, k + row * ldk + (size_t)hq * dk + cc, ok);
                if (PER_CHANNEL) ls_cp_async_16(w_s(buf, tt) + c, w + row * ldw + (size_t)h * dk + cc, ok);
            }
        } else
        for (int e = threadIdx.x; e < TB * DKP; e += LS_THREADS) {
            const int tt = e / DKP, c = e % DKP;
            const bool ok = tt < nt && c < dk;
            const size_t row = (size_t)(base + (ok ? tt : 0));
            const int cc = ok ? c : 0;
            if (MODE != 1) ls_cp_async_4(q_s(buf, tt) + c, q + row * ldq + (size_t)hq * dk + cc, ok);
            ls_cp_async_4(k_s(buf, tt) + c, k + row * ldk + (size_t)hq * dk + cc, ok);
            if (PER_CHANNEL) ls_cp_async_4(w_s(buf, tt) + c, w + row * ldw + (size_t)h * dk + cc, ok);
        }
        for (int e = threadIdx.x; e < TB * LS_COLS; e += LS_THREADS) {
            const int tt = e / LS_COLS, cc = e % LS_COLS, jj = blockIdx.x * LS_COLS + cc;
            const bool ok = tt < nt && jj < dv;
            ls_cp_async_4(v_s(buf, tt) + cc, v + (size_t)(base + (ok ? tt : 0)) * ldv + (size_t)h * dv + (ok ? jj : 0), ok);
        }
        if (threadIdx.x < TB) {
            const int tt = threadIdx.x;
            const bool ok = tt < nt;
            const size_t row = (size_t)(base + (ok ? tt : 0));
            if (!PER_CHANNEL) ls_cp_async_4(w_s(buf, tt), w + row * ldw + h, ok);
            if (scaled) ls_cp_async_4(f_s(buf) + tt, v_scale + row * heads + h, ok);
        }
    };

    // every turn commits one group, empty or not, so that "all but the last STAGES - 1 groups" is always this chunk
    for (int st = 0; st < STAGES - 1; ++st) {
        if (row0 + st * TB < row1) stage(st, row0 + st * TB);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    int buf = 0;
    for (int base = row0; base < row1; base += TB, buf = (buf + 1 == STAGES ? 0 : buf + 1)) {
        const int nt = min(TB, row1 - base);
        const int ahead = base + (STAGES - 1) * TB;
        if (ahead < row1) stage(buf == 0 ? STAGES - 1 : buf - 1, ahead);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1));
        __syncthreads();
        float part[TB];     // this lane's share of each token's output
        auto token = [&](int tt) {
            const float vv = scaled ? v_s(buf, tt)[col] * f_s(buf)[tt] : v_s(buf, tt)[col];
            const float wh = PER_CHANNEL ? 0.f : w_s(buf, tt)[0];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < C / 4; ++i4) {
                const int c4 = (i4 * LS_LANES + lane) * 4;
                float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (MODE != 1) q4 = *reinterpret_cast<const float4*>(q_s(buf, tt) + c4);
                const float4 k4 = *reinterpret_cast<const float4*>(k_s(buf, tt) + c4);
                float4 w4 = make_float4(wh, wh, wh, wh);
                if (PER_CHANNEL) w4 = *reinterpret_cast<const float4*>(w_s(buf, tt) + (PER_CHANNEL ? c4 : 0));
                const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w}, wa[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = i4 * 4 + e;
                    const float kv = ka[e] * vv;
                    if (MODE == 1) {
                        S[i] = fmaf(wa[e], S[i], kv);
                        if (track) P[i] *= wa[e];
                    } else if (BONUS) {
                        acc[e] = fmaf(qa[e], fmaf(U[i], kv, S[i]), acc[e]);
                        S[i] = fmaf(wa[e], S[i], kv);
                    } else {
                        S[i] = fmaf(wa[e], S[i], kv);
                        acc[e] = fmaf(qa[e], S[i], acc[e]);
                    }
                }
            }
            return (acc[0] + acc[1]) + (acc[2] + acc[3]);
        };
        if (nt == TB) {     // a full chunk, unrolled: only the state chains its tokens
#pragma unroll
            for (int tt = 0; tt < TB; ++tt) part[tt] = token(tt);
        } else {
#pragma unroll
            for (int tt = 0; tt < TB; ++tt) part[tt] = tt < nt ? token(tt) : 0.f;
        }
        // The eight lanes of a column sum their shares of the eight tokens in three exchanges (4 + 2 + 1 shuffles), each
        // lane keeping half of what it held: lane l ends with token l's output. The pairs are those of a butterfly over
        // one token's shares (lane ^ 4, then ^ 2, then ^ 1), whatever the chunk holds.
        if (MODE != 1) {
            const bool up4 = (lane & 4) != 0, up2 = (lane & 2) != 0, up1 = (lane & 1) != 0;
            float h4[4], h2[2];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float recv = __shfl_xor_sync(0xffffffffu, up4 ? part[t] : part[t + 4], 4);
                h4[t] = (up4 ? part[t + 4] : part[t]) + recv;
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const float recv = __shfl_xor_sync(0xffffffffu, up2 ? h4[t] : h4[t + 2], 2);
                h2[t] = (up2 ? h4[t + 2] : h4[t]) + recv;
            }
            const float recv = __shfl_xor_sync(0xffffffffu, up1 ? h2[0] : h2[1], 1);
            const float total = (up1 ? h2[1] : h2[0]) + recv;
            if (lane < nt && j < dv) o[(size_t)(base + lane) * ldo + (size_t)h * dv + j] = total * q_scale;
        }
        __syncthreads();        // the chunk has been walked: its buffer may be filled again
    }
    float* to = MODE == 0 ? srow : (MODE == 1 ? seg_row + elems : (last ? srow : nullptr));     // a segment's end is the next one's entry
    if (j < dv && to != nullptr) {
#pragma unroll
        for (int i = 0; i < C; ++i) {
            const int c = ((i >> 2) * LS_LANES + lane) * 4 + (i & 3);
            if (c < dk) to[c] = S[i];
        }
    }
    if (MODE == 1 && track) {
        float* pd = seg_decay + (((size_t)req * n_seg + seg) * heads + h) * (PER_CHANNEL ? dk : 1);
        if (PER_CHANNEL) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                const int c = ((i >> 2) * LS_LANES + lane) * 4 + (i & 3);
                if (c < dk) pd[c] = P[MODE == 1 ? i : 0];
            }
        } else if (lane == 0) {
            pd[0] = P[0];
        }
    }
}

// Entry states of a request's segments: seg_state[0] = the slot's state, seg_state[s + 1] = decay(s) * seg_state[s] +
// (what the first walk left there: segment s walked from zero). One thread per state element.
__global__ void __launch_bounds__(256)
ls_combine_kernel(const float* __restrict__ state, long long state_ld, int state_off, const int* __restrict__ q_start,
                  const int* __restrict__ slots, float* __restrict__ seg_state, const float* __restrict__ seg_decay, int n_req,
                  int n_seg, int seg_len, int heads, int dk, int dv, int per_channel) {
    const size_t elems = (size_t)heads * dv * dk;
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)n_req * elems) return;
    const int req = (int)(e / elems);
    const size_t x = (size_t)(e % elems);
    const int c = (int)(x % dk), h = (int)(x / ((size_t)dv * dk));
    const int len = q_start[req + 1] - q_start[req];
    const int segs = (len + seg_len - 1) / seg_len;
    float S = state[(long long)slots[req] * state_ld + state_off + x];
    float* base = seg_state + (size_t)req * n_seg * elems + x;
    base[0] = S;
    for (int s = 0; s + 1 < segs; ++s) {
        const float p = per_channel ? seg_decay[(((size_t)req * n_seg + s) * heads + h) * dk + c] : seg_decay[((size_t)req * n_seg + s) * heads + h];
        S = fmaf(p, S, base[(size_t)(s + 1) * elems]);
        base[(size_t)(s + 1) * elems] = S;
    }
}

// The number of floats of scratch that the walk in segments wants for these sizes (states, then decay products).
NIB_API long long nib_linear_state_scan_scratch(int n_req, int n_seg, int heads, int dk, int dv) {
    return (long long)n_req * n_seg * heads * ((long long)dv * dk + dk);
}

// n_seg <= 1: every request's tokens in order, one block per (request, head, 16 value columns). n_seg > 1 (long
// prompts): segments of seg_len tokens side by side (see the kernel); scratch holds nib_linear_state_scan_scratch floats.
NIB_API int nib_linear_state_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* w, int ldw,
                                  int w_per_channel, const float* bonus, const float* v_scale, float* state, long long state_ld,
                                  int state_off, const int* q_start, const int* slots, float* o, int ldo, int n_req, int heads,
                                  int kq_heads, int dk, int dv, float q_scale, int n_seg, int seg_len, float* scratch,
                                  cudaStream_t stream) {
    NIB_REQUIRE(heads > 0 && kq_heads > 0 && heads % kq_heads == 0, "linear_state_scan: %d heads do not share %d key heads", heads, kq_heads);
    NIB_REQUIRE(dk > 0 && dk <= 256 && dv > 0, "linear_state_scan: key size %d is outside 1..256", dk);
    NIB_REQUIRE(n_seg <= 1 || (scratch != nullptr && seg_len > 0 && seg_len % 8 == 0), "linear_state_scan: segments need scratch and a length that is a multiple of 8");
    if (n_req <= 0) return 0;
    const bool cut = n_seg > 1;
    auto aligned = [](const void* p, int ld) { return ((uintptr_t)p & 15) == 0 && ld % 4 == 0; };
    const int vec = (dk % 4 == 0 && aligned(q, ldq) && aligned(k, ldk) && (!w_per_channel || aligned(w, ldw))) ? 1 : 0;
    float* seg_state = scratch;
    float* seg_decay = cut ? scratch + (size_t)n_req * n_seg * heads * dv * dk : nullptr;
    const dim3 block(LS_THREADS);
#define NIB_LS_LAUNCH4(C, PC, B, MODE)                                                                                              \
    do {                                                                                                                            \
        static bool configured = false;                                                                                             \
        if (!configured) {                                                                                                          \
            NIB_CUDA(cudaFuncSetAttribute(linear_state_scan_kernel<C, PC, B, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                          LsLayout<C, PC>::BYTES));                                                                 \
            configured = true;                                                                                                      \
        }                                                                                                                           \
        const dim3 grid(ceil_div(dv, LS_COLS), heads, n_req * (MODE == 0 ? 1 : n_seg));                                             \
        linear_state_scan_kernel<C, PC, B, MODE><<<grid, block, LsLayout<C, PC>::BYTES, stream>>>(                                  \
            q, ldq, k, ldk, v, ldv, w, ldw, bonus, v_scale, state, state_ld, state_off, q_start, slots, o, ldo, heads, kq_heads,    \
            dk, dv, q_scale, n_seg, seg_len, seg_state, seg_decay, vec);                                                            \
        NIB_LAUNCH_CHECK();                                                                                                         \
    } while (0)
#define NIB_LS_LAUNCH3(C, PC, B)                                                                                                    \
    do {                                                                                                                            \
        if (!cut) {                                                                                                                 \
            NIB_LS_LAUNCH4(C, PC, B, 0);                                                                                            \
        } else {                                                                                                                    \
            NIB_LS_LAUNCH4(C, PC, false, 1);                                                                                        \
            ls_combine_kernel<<<ceil_div((long long)n_req * heads * dv * dk, 256), 256, 0, stream>>>(                               \
                state, state_ld, state_off, q_start, slots, seg_state, seg_decay, n_req, n_seg, seg_len, heads, dk, dv, PC ? 1 : 0); \
            NIB_LAUNCH_CHECK();                                                                                                     \
            NIB_LS_LAUNCH4(C, PC, B, 2);                                                                                            \
        }                                                                                                                           \
    } while (0)
#define NIB_LS_LAUNCH(C)                                            \
    do {                                                            \
        if (w_per_channel && bonus != nullptr) NIB_LS_LAUNCH3(C, true, true);   \
        else if (w_per_channel) NIB_LS_LAUNCH3(C, true, false);     \
        else if (bonus != nullptr) NIB_LS_LAUNCH3(C, false, true);  \
        else NIB_LS_LAUNCH3(C, false, false);                       \
    } while (0)
    if (dk <= 32) NIB_LS_LAUNCH(4);
    else if (dk <= 64) NIB_LS_LAUNCH(8);
    else if (dk <= 128) NIB_LS_LAUNCH(16);
    else NIB_LS_LAUNCH(32);
#undef NIB_LS_LAUNCH
#undef NIB_LS_LAUNCH3
#undef NIB_LS_LAUNCH4
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

// Both in one launch for steps of a few tokens per request (a decode step): one thread per (request, channel) walks the
// request's tokens with the history in registers, then writes the history back. The same arithmetic per output as
// conv_tokens_kernel (taps added in ascending order from the bias).
constexpr int CONV_STEP_MAX_TAPS = 16;

__global__ void __launch_bounds__(256)
conv_step_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias, int act,
                 float* __restrict__ state, long long state_ld, int state_off, const int* __restrict__ q_start,
                 const int* __restrict__ slots, float* __restrict__ y, int ldy, int n_req, int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)n_req * width) return;
    const int r = (int)(e / width), c = (int)(e % width);
    const int first = q_start[r], len = q_start[r + 1] - first;
    float* hist = taps > 1 ? state + (long long)slots[r] * state_ld + state_off : nullptr;
    float win[CONV_STEP_MAX_TAPS - 1], wt[CONV_STEP_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_STEP_MAX_TAPS; ++j) {
        wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        if (j < CONV_STEP_MAX_TAPS - 1) win[j] = j < taps - 1 ? hist[(size_t)j * width + c] : 0.f;
    }
    const float b = bias != nullptr ? bias[c] : 0.f;
    for (int i = 0; i < len; ++i) {
        const float u = x[(size_t)(first + i) * ldx + c];
        float acc = b;
#pragma unroll
        for (int j = 0; j < CONV_STEP_MAX_TAPS - 1; ++j)
            if (j < taps - 1) acc = fmaf(wt[j], win[j], acc);
#pragma unroll
        for (int j = 0; j < CONV_STEP_MAX_TAPS; ++j)
            if (j == taps - 1) acc = fmaf(wt[j], u, acc);
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        y[(size_t)(first + i) * ldy + c] = acc;
#pragma unroll
        for (int j = 0; j < CONV_STEP_MAX_TAPS - 1; ++j) {
            if (j < taps - 2) win[j] = win[j + 1 < CONV_STEP_MAX_TAPS - 1 ? j + 1 : j];
            else if (j == taps - 2) win[j] = u;
        }
    }
#pragma unroll
    for (int j = 0; j < CONV_STEP_MAX_TAPS - 1; ++j)
        if (j < taps - 1) hist[(size_t)j * width + c] = win[j];
}

NIB_API int nib_conv_step(const float* x, int ldx, const float* w, const float* bias, int act, float* state, long long state_ld,
                          int state_off, const int* q_start, const int* slots, float* y, int ldy, int n_req, int width, int taps,
                          cudaStream_t stream) {
    NIB_REQUIRE(n_req >= 0 && width > 0 && taps >= 1 && taps <= CONV_STEP_MAX_TAPS && (taps == 1 || state != nullptr),
                "conv_step: bad sizes, more than %d taps, or no state", CONV_STEP_MAX_TAPS);
    if (n_req == 0) return 0;
    NIB_CUDA(launch_pdl(conv_step_kernel, dim3(ceil_div((long long)n_req * width, 256)), dim3(256), (size_t)0, stream, x, ldx, w, bias, act,
                        state, state_ld, state_off, q_start, slots, y, ldy, n_req, width, taps));
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
