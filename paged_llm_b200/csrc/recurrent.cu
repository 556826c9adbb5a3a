// Mixers that carry a state of fixed size from token to token, in float32:
//
//  * a causal convolution per channel over a projection's columns (bias on the input, bias on the output, no
//    activation or silu), whose last taps-1 inputs are part of the request's state;
//  * a real-gated linear recurrence per channel:
//        a = exp(rate * sigmoid(g_r)),   S_t = a S_(t-1) + sqrt(1 - a^2) * sigmoid(g_i) * u_t,   out = S_t * gelu_tanh(y_t)
//  * gated linear attention, a matrix state per head with a decay per key channel:
//        alpha = exp(log_sigmoid(z) / tau),   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
//  * the gated delta rule, a matrix state per head:
//        S <- g S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T q
//  * the norm of each head's output over its value size, times silu(gate).
//
// Every request of the step brings its next tokens (one when it decodes, many in a prompt portion); its state lives
// in a slot of [slots, state_stride] floats.  The recurrences run in the order of the tokens with a fixed order of
// sums, so what a position gets does not depend on how the prompt was cut or on the batch.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
// log(sigmoid(v)) without overflow: min(v, 0) - log1p(exp(-|v|))
__device__ __forceinline__ float log_sigmoid_f(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

// ------------------------------------------------------------------ causal convolution
// grid: (requests, channel blocks of 32, token chunks of CONV_TOK).  Input of channel c at token t:
// in[t, col0 + c] + b_in[col0 + c].  The block of chunk 0 is the only one that reads the request's old inputs (the
// state's first (taps-1) * C floats, [taps-1][C]), and it alone writes the new ones, after a barrier.
constexpr int CONV_TOK = 64;

template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ in, int ld, int col0, int C,
                                                          const float* __restrict__ b_in, const float* __restrict__ cw,
                                                          const float* __restrict__ cb, int taps, float* __restrict__ state,
                                                          long long state_stride, const int* __restrict__ cu_q,
                                                          const int* __restrict__ slots, float* __restrict__ u,
                                                          T* __restrict__ u_low, int act) {
    const int s = blockIdx.x;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    const int t_lo = blockIdx.z * CONV_TOK, t_hi = min(nq, t_lo + CONV_TOK);
    if (slot < 0 || t_lo >= nq) return;
    const int lane_c = threadIdx.x & 31, lane_t = threadIdx.x >> 5;
    const int c = blockIdx.y * 32 + lane_c;
    const bool ok = c < C;
    float* st = state + (size_t)slot * state_stride;
    const int hist = taps - 1;
    const float bi = ok && b_in != nullptr ? __ldg(b_in + col0 + c) : 0.f;
    const T* col = in + (size_t)q0 * ld + col0 + (ok ? c : 0);
    auto input = [&](int src) { return src >= 0 ? to_float(col[(size_t)src * ld]) + bi : st[(size_t)(hist + src) * C + c]; };
    if (ok) {
        const float bias = cb != nullptr ? __ldg(cb + c) : 0.f;
        for (int t = t_lo + lane_t; t < t_hi; t += 8) {
            float acc = bias;
            for (int k = 0; k < taps; ++k) acc = fmaf(__ldg(cw + (size_t)c * taps + k), input(t - hist + k), acc);
            if (act == 1) acc = acc / (1.0f + expf(-acc));          // silu
            u[(size_t)(q0 + t) * C + c] = acc;
            if (u_low != nullptr) u_low[(size_t)(q0 + t) * C + c] = from_float<T>(acc);
        }
    }
    if (blockIdx.z != 0) return;
    __syncthreads();                                                // every read of the old inputs is done
    if (ok && lane_t == 0) {
        // the last taps-1 inputs of [old inputs ; this step's inputs]: in place from the front, since entry j
        // reads old entry j + nq > j or a new input
        for (int j = 0; j < hist; ++j) {
            const int src = nq + j - hist;
            st[(size_t)j * C + c] = src >= 0 ? to_float(col[(size_t)src * ld]) + bi : st[(size_t)(j + nq) * C + c];
        }
    }
}

// `max_tokens`: no request of the step brings more.  u: [T, C] float32; u_low: the same in `dtype`, or null.
PL_EXPORT int pl_causal_conv(const void* in, int dtype, int ld, int col0, int C, const float* b_in, const float* cw,
                             const float* cb, int taps, float* state, long long state_stride, const int* cu_q,
                             const int* slots, int num_seqs, int max_tokens, float* u, void* u_low, int act,
                             cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(act == 0 || act == 1, "causal_conv: unknown activation %d", act);
    PL_REQUIRE(C > 0 && taps >= 1 && taps <= CONV_TOK && max_tokens >= 1 && col0 >= 0 && col0 + C <= ld,
               "causal_conv: bad sizes C=%d taps=%d col0=%d ld=%d", C, taps, col0, ld);
    const dim3 grid(num_seqs, (C + 31) / 32, (max_tokens + CONV_TOK - 1) / CONV_TOK);
    PL_REQUIRE(grid.z <= 65535 && grid.y <= 65535, "causal_conv: %d tokens, %d channels in a step", max_tokens, C);
    if (dtype == PL_F32)
        causal_conv_kernel<float><<<grid, 256, 0, stream>>>((const float*)in, ld, col0, C, b_in, cw, cb, taps, state, state_stride,
                                                            cu_q, slots, u, (float*)u_low, act);
    else if (dtype == PL_BF16)
        causal_conv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, ld, col0, C, b_in, cw, cb, taps,
                                                                    state, state_stride, cu_q, slots, u, (__nv_bfloat16*)u_low, act);
    else
        return pl_fail("causal_conv: unknown dtype %d", dtype);
    PL_LAUNCHED("causal_conv");
    return 0;
}

// ------------------------------------------------------------------ real-gated linear recurrence
// grid: (requests, channel blocks).  Threads: CH = 256 / TL channel lanes x TL token lanes.  A tile of TL * SEG
// tokens is worked on at once: token lane j takes SEG consecutive tokens, forms their decays a and drives
// b = sqrt(1 - a^2) * sigmoid(g_i) * u (kept in registers) and the pair (A, B) that carries a state across its
// tokens (S -> A S + B); the pairs of the lanes in front, applied in order to the state at the start of the tile,
// give the lane its own start, from which it runs its tokens again and writes S_t * gelu_tanh(y_t + bias).
// gates: [T, blocks * 2 * bw] float32, per block [recurrence gate: bw | input gate: bw], biases `b_gates` the
// same; channel c belongs to block c / bw.  The state S of a request: `state_off` floats into its slot.
constexpr int REC_SEG = 8;

// The decays and drives of all tokens at once, in place: gates[t, r-part of c] <- a, gates[t, i-part of c] <- b.  A long
// prompt's transcendental work is spread over the whole device here, and the scan behind it only multiplies and adds.
__global__ void __launch_bounds__(256) recurrence_prepare_kernel(float* __restrict__ gates, const float* __restrict__ b_gates,
                                                                 const float* __restrict__ u, const float* __restrict__ rate,
                                                                 int C, int bw, long long n) {
    const int G = (C / bw) * 2 * bw;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / C;
        const int c = (int)(i - row * C);
        const int blk = c / bw, j = c - blk * bw;
        const int gr = blk * 2 * bw + j, gi = gr + bw;
        const float r = sigmoid_f(gates[row * G + gr] + __ldg(b_gates + gr)), in = sigmoid_f(gates[row * G + gi] + __ldg(b_gates + gi));
        const float la = __ldg(rate + c) * r;
        gates[row * G + gr] = expf(la);
        gates[row * G + gi] = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f)) * in * u[i];
    }
}

template <typename T, int TL, bool PRE>
__global__ void __launch_bounds__(256) gated_recurrence_kernel(const float* __restrict__ gates, const float* __restrict__ b_gates,
                                                               const float* __restrict__ u, const T* __restrict__ yx, int ld,
                                                               const float* __restrict__ b_y, const float* __restrict__ rate,
                                                               int C, int bw, float* __restrict__ state, long long state_stride,
                                                               long long state_off, const int* __restrict__ cu_q,
                                                               const int* __restrict__ slots, T* __restrict__ out) {
    constexpr int CH = 256 / TL;
    __shared__ float carry[2][TL][CH];
    const int s = blockIdx.x;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    const int lane_c = threadIdx.x % CH, lane_t = threadIdx.x / CH;
    const int c = blockIdx.y * CH + lane_c;
    const bool ok = c < C;
    const int cc = ok ? c : 0;
    const int blk = cc / bw, j = cc - blk * bw;
    const int gr = blk * 2 * bw + j, gi = gr + bw, G = (C / bw) * 2 * bw;
    const float br = __ldg(b_gates + gr), bi = __ldg(b_gates + gi), rt = __ldg(rate + cc), by = __ldg(b_y + cc);
    float* sp = state + (size_t)slot * state_stride + state_off + cc;
    float S0 = ok ? *sp : 0.f;                                      // the state at the start of the tile
    for (int t0 = 0; t0 < nq; t0 += TL * REC_SEG) {
        const int ta = t0 + lane_t * REC_SEG;
        float a[REC_SEG], b[REC_SEG];
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int i = 0; i < REC_SEG; ++i) {
            a[i] = 1.f, b[i] = 0.f;
            if (PRE) {
                if (ok && ta + i < nq) {
                    const size_t row = (size_t)(q0 + ta + i);
                    a[i] = gates[row * G + gr], b[i] = gates[row * G + gi];
                }
            } else if (ok && ta + i < nq) {
                const size_t row = (size_t)(q0 + ta + i);
                const float r = sigmoid_f(gates[row * G + gr] + br), in = sigmoid_f(gates[row * G + gi] + bi);
                // 1 - a^2 = -expm1(2 log a): formed from the exponent, so that nothing cancels where a is close to 1
                const float la = rt * r;
                a[i] = expf(la);
                b[i] = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f)) * in * u[row * C + c];
            }
            A *= a[i];
            B = fmaf(a[i], B, b[i]);
        }
        float S = S0;
        if (TL > 1) {
            carry[0][lane_t][lane_c] = A;
            carry[1][lane_t][lane_c] = B;
            __syncthreads();
            float Sj = S0;
#pragma unroll
            for (int l = 0; l < TL; ++l) {
                if (l == lane_t) S = Sj;
                Sj = fmaf(carry[0][l][lane_c], Sj, carry[1][l][lane_c]);
            }
            S0 = Sj;                                                // every lane knows the state behind the tile
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < REC_SEG; ++i) {
            S = fmaf(a[i], S, b[i]);
            if (ok && ta + i < nq) {
                const size_t row = (size_t)(q0 + ta + i);
                out[row * C + c] = from_float<T>(S * gelu_tanh_f(to_float(yx[row * ld + c]) + by));
            }
        }
        if (TL == 1) S0 = S;
    }
    if (ok && lane_t == 0) *sp = S0;
}

// yx: the projection's rows [y: C | ...] with row stride ld in `dtype`; out: [T, C] in `dtype`.  With more than a few tokens
// in a request the gates [total_tokens, 2C] are overwritten by the decays and drives (recurrence_prepare_kernel).
PL_EXPORT int pl_gated_recurrence(float* gates, const float* b_gates, const float* u, const void* yx, int dtype, int ld,
                                  const float* b_y, const float* rate, int C, int blocks, float* state,
                                  long long state_stride, long long state_off, const int* cu_q, const int* slots,
                                  int num_seqs, int max_tokens, long long total_tokens, void* out, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(C > 0 && blocks > 0 && C % blocks == 0 && ld >= C, "gated_recurrence: bad sizes C=%d blocks=%d ld=%d", C, blocks, ld);
    const int bw = C / blocks;
    const bool few = max_tokens <= 2 * REC_SEG;
    const bool many = max_tokens > 32 * REC_SEG;                     // long prompts: more token lanes, more blocks
    const int CH = few ? 256 : many ? 8 : 32;
    const dim3 grid(num_seqs, (C + CH - 1) / CH);
    PL_REQUIRE(grid.y <= 65535, "gated_recurrence: %d channels", C);
#define PL_REC(TT, L)                                                                                                      \
    gated_recurrence_kernel<TT, L, L != 1><<<grid, 256, 0, stream>>>(gates, b_gates, u, (const TT*)yx, ld, b_y, rate, C, bw,   \
                                                                     state, state_stride, state_off, cu_q, slots, (TT*)out)
    if (!few) {
        PL_REQUIRE(total_tokens > 0, "gated_recurrence: %lld tokens", total_tokens);
        const long long n = total_tokens * C, blocks = (n + 255) / 256;
        recurrence_prepare_kernel<<<(unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16), 256, 0, stream>>>(gates, b_gates, u, rate,
                                                                                                          C, bw, n);
        PL_LAUNCHED("recurrence_prepare");
    }
    if (dtype == PL_F32) {
        if (few) PL_REC(float, 1); else if (!many) PL_REC(float, 8); else PL_REC(float, 32);
    } else if (dtype == PL_BF16) {
        if (few) PL_REC(__nv_bfloat16, 1); else if (!many) PL_REC(__nv_bfloat16, 8); else PL_REC(__nv_bfloat16, 32);
    } else {
        return pl_fail("gated_recurrence: unknown dtype %d", dtype);
    }
#undef PL_REC
    PL_LAUNCHED("gated_recurrence");
    return 0;
}

// ------------------------------------------------------------------ gated linear attention, the recurrence
// A column v of a head's state (its d values over the key channels) is independent of the other columns: GLA_LANES
// lanes share it, each holding NPER of the key channels in registers (gla_channel), and a block of 128 threads runs 16
// columns.  The tokens' q (scaled), k, decay and v come into shared memory sixteen (the widest heads: eight) tokens at
// a time.  Per token a lane does 2 NPER multiply-adds and the lanes' parts of the output are summed by shuffles in a
// fixed order.  The decay is alpha = exp(log_sigmoid(z + bias) / tau) in float32: formed by every block for its head
// (z_bias given), or beforehand for all tokens at once (gla_decay_kernel, z_bias null: z holds alpha).
//
// Whole requests (seg_len 0), grid (requests, heads, column blocks): a block runs all tokens of its request.
// Long prompts (seg_len > 0), grid (requests * segments, heads, column blocks), two launches.  A request's tokens are
// cut into segments of seg_len.  First launch: segment 0 runs from the request's state and writes its outputs; every
// later segment but the last runs from a zero state without outputs and leaves the state L it ends in and the product
// D of its decays.  Second launch: segment p >= 1 starts from L_0 carried through the segments in between
// (S <- D_j S + L_j) and writes its outputs; the last one stores the request's state.  A request of one segment is
// done by the first launch alone.  L and D of the segment that starts at row r are entry r / seg_len of `seg_state`
// (per column) and `seg_decay` (per head and key channel; full segments do not overlap, so neither do their entries).
// proj: rows [q: H*d | k: H*d | v: H*dv | ...] in T; z: [T, H*d] float32; state: [H][dv][d] floats per slot;
// o: [T, H*dv] float32.
constexpr int GLA_TOK_MAX = 16;
constexpr int GLA_LANES = 8;
constexpr int GLA_COLS = 128 / GLA_LANES;
constexpr int GLA_SEG = 128;                                        // tokens in a segment of a long prompt

__global__ void __launch_bounds__(256) gla_decay_kernel(float* __restrict__ z, const float* __restrict__ z_bias, int K,
                                                        float inv_tau, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        z[i] = expf(log_sigmoid_f(z[i] + __ldg(z_bias + (int)(i % K))) * inv_tau);
}

// The key channel that value i of lane `lane` stands for.  Wide heads (NPER a multiple of 4): four consecutive channels
// at a time, so that a lane reads its q, k and decay from shared memory, and its state from memory, 16 bytes at once
// and the eight lanes of a column cover 128 consecutive bytes.  Narrow heads: channel lane + 8 i.
template <int NPER>
__device__ __forceinline__ int gla_channel(int lane, int i) {
    return NPER % 4 == 0 ? (i >> 2) * (GLA_LANES * 4) + lane * 4 + (i & 3) : lane + GLA_LANES * i;
}

template <typename T, int NPER>
__global__ void __launch_bounds__(128) gla_scan_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ z,
                                                       const float* __restrict__ z_bias, int H, int d, int dv, float inv_tau,
                                                       float q_scale, float* __restrict__ state, long long state_stride,
                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                       float* __restrict__ o, int seg_len, int segs, int second,
                                                       float* __restrict__ seg_state, float* __restrict__ seg_decay) {
    constexpr int ROW = GLA_LANES * NPER;                           // a token's q (or k, or decay), zeros from d on
    constexpr int GLA_TOK = NPER > 16 ? GLA_TOK_MAX / 2 : GLA_TOK_MAX;     // (static shared memory ends at 48 KB)
    __shared__ __align__(16) float qs[GLA_TOK][ROW], ks[GLA_TOK][ROW], as[GLA_TOK][ROW], vs[GLA_TOK][GLA_COLS];
    const int s = seg_len > 0 ? blockIdx.x / segs : blockIdx.x;
    const int h = blockIdx.y, v0 = blockIdx.z * GLA_COLS;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    int p = 0, P = 1, t_begin = 0, t_end = nq;
    if (seg_len > 0) {
        P = (nq + seg_len - 1) / seg_len;
        p = blockIdx.x % segs + (second ? 1 : 0);
        if (p >= P || (!second && p > 0 && p == P - 1)) return;     // (the last segment belongs to the second launch)
        t_begin = p * seg_len;
        t_end = min(nq, t_begin + seg_len);
    }
    const bool last = p == P - 1;
    const bool emit = second || p == 0;
    // (the product of a segment's decays is the same for every column: one column of the head's first block forms it)
    const bool track = !second && p > 0 && blockIdx.z == 0 && threadIdx.x < GLA_LANES;
    const int tid = threadIdx.x, lane = tid & (GLA_LANES - 1), col = tid / GLA_LANES;
    const int v = v0 + col;
    const bool ok = v < dv;
    const size_t col_off = ((size_t)h * dv + (ok ? v : 0)) * d, seg_stride = (size_t)H * dv * d;
    float* sp = state + (size_t)slot * state_stride + col_off;
    float S[NPER], Dp[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = gla_channel<NPER>(lane, i);
        Dp[i] = 1.f;
        S[i] = 0.f;
        if (ok && n < d) {
            if (p == 0) S[i] = sp[n];
            else if (second) S[i] = seg_state[(size_t)(q0 / seg_len) * seg_stride + col_off + n];
        }
    }
    if (second && ok) {
        // (segment by segment, all of the lane's values at once: their loads are independent of each other)
        for (int j = 1; j < p; ++j) {
            const size_t entry = (size_t)((q0 + j * seg_len) / seg_len);
            const float* Lj = seg_state + entry * seg_stride + col_off;
            const float* Dj = seg_decay + (entry * H + h) * d;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                const int n = gla_channel<NPER>(lane, i);
                if (n < d) S[i] = fmaf(Dj[n], S[i], Lj[n]);
            }
        }
    }
    const T* q_src = proj + (size_t)h * d;
    const T* k_src = proj + (size_t)H * d + (size_t)h * d;
    const T* v_src = proj + (size_t)2 * H * d + (size_t)h * dv + v0;
    const float* z_src = z + (size_t)h * d;
    for (int t0 = t_begin; t0 < t_end; t0 += GLA_TOK) {
        const int nt = min(GLA_TOK, t_end - t0);
        for (int i = tid; i < GLA_TOK * ROW; i += 128) {
            const int t = i / ROW, n = i - t * ROW;
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (t < nt && n < d) {
                const size_t row = (size_t)(q0 + t0 + t);
                qv = to_float(q_src[row * ld + n]) * q_scale;
                kv = to_float(k_src[row * ld + n]);
                av = z_src[row * (size_t)H * d + n];
                if (z_bias != nullptr) av = expf(log_sigmoid_f(av + __ldg(z_bias + h * d + n)) * inv_tau);
            }
            qs[t][n] = qv, ks[t][n] = kv, as[t][n] = av;
        }
        for (int i = tid; i < GLA_TOK * GLA_COLS; i += 128) {
            const int t = i / GLA_COLS, c = i - t * GLA_COLS;
            vs[t][c] = t < nt && v0 + c < dv ? to_float(v_src[(size_t)(q0 + t0 + t) * ld + c]) : 0.f;
        }
        __syncthreads();
        if (emit) {
#pragma unroll 4
            for (int t = 0; t < GLA_TOK; ++t) {
                if (t < nt) {                                       // (uniform over the block)
                    const float vv = vs[t][col];
                    float acc0 = 0.f, acc1 = 0.f;
                    if (NPER % 4 == 0) {
#pragma unroll
                        for (int i4 = 0; i4 < NPER / 4; ++i4) {
                            const int n = i4 * (GLA_LANES * 4) + lane * 4;
                            const float4 a4 = *reinterpret_cast<const float4*>(&as[t][n]);
                            const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][n]);
                            const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][n]);
                            float* S4 = S + i4 * 4;
                            S4[0] = fmaf(a4.x, S4[0], k4.x * vv), S4[1] = fmaf(a4.y, S4[1], k4.y * vv);
                            S4[2] = fmaf(a4.z, S4[2], k4.z * vv), S4[3] = fmaf(a4.w, S4[3], k4.w * vv);
                            acc0 = fmaf(S4[0], q4.x, acc0), acc1 = fmaf(S4[1], q4.y, acc1);
                            acc0 = fmaf(S4[2], q4.z, acc0), acc1 = fmaf(S4[3], q4.w, acc1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < NPER; ++i) {
                            const int n = lane + GLA_LANES * i;
                            S[i] = fmaf(as[t][n], S[i], ks[t][n] * vv);
                            if (i & 1) acc1 = fmaf(S[i], qs[t][n], acc1); else acc0 = fmaf(S[i], qs[t][n], acc0);
                        }
                    }
                    float acc = acc0 + acc1;
#pragma unroll
                    for (int m = GLA_LANES / 2; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
                    if (ok && lane == 0) o[(size_t)(q0 + t0 + t) * H * dv + (size_t)h * dv + v] = acc;
                }
            }
        } else {
#pragma unroll 4
            for (int t = 0; t < GLA_TOK; ++t) {
                if (t < nt) {
                    const float vv = vs[t][col];
                    if (NPER % 4 == 0) {
#pragma unroll
                        for (int i4 = 0; i4 < NPER / 4; ++i4) {
                            const int n = i4 * (GLA_LANES * 4) + lane * 4;
                            const float4 a4 = *reinterpret_cast<const float4*>(&as[t][n]);
                            const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][n]);
                            float* S4 = S + i4 * 4;
                            S4[0] = fmaf(a4.x, S4[0], k4.x * vv), S4[1] = fmaf(a4.y, S4[1], k4.y * vv);
                            S4[2] = fmaf(a4.z, S4[2], k4.z * vv), S4[3] = fmaf(a4.w, S4[3], k4.w * vv);
                            if (track) Dp[i4 * 4] *= a4.x, Dp[i4 * 4 + 1] *= a4.y, Dp[i4 * 4 + 2] *= a4.z, Dp[i4 * 4 + 3] *= a4.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < NPER; ++i) {
                            const int n = lane + GLA_LANES * i;
                            S[i] = fmaf(as[t][n], S[i], ks[t][n] * vv);
                            if (track) Dp[i] *= as[t][n];
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    if (!ok) return;
    if (last) {
#pragma unroll
        for (int i = 0; i < NPER; ++i)
            if (gla_channel<NPER>(lane, i) < d) sp[gla_channel<NPER>(lane, i)] = S[i];
    } else if (!second) {
        const size_t e = (size_t)((q0 + t_begin) / seg_len) * seg_stride + col_off;
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = gla_channel<NPER>(lane, i);
            if (n < d) {
                seg_state[e + n] = S[i];
                if (track) seg_decay[((size_t)((q0 + t_begin) / seg_len) * H + h) * d + n] = Dp[i];
            }
        }
    }
}

// `max_tokens`: no request of the step brings more; `total_tokens`: rows of proj, z and o.  With max_tokens of at least two
// segments the caller gives `seg_state` and `seg_decay`, each ceil(total_tokens / GLA_SEG) * H * dv * d floats
// (pl_gla_segment() tells the segment's length); z is then overwritten by the decays.
PL_EXPORT int pl_gla_segment() { return GLA_SEG; }

PL_EXPORT int pl_gla_scan(const void* proj, int dtype, int ld, float* z, const float* z_bias, int H, int d, int dv,
                          float tau, float q_scale, float* state, long long state_stride, const int* cu_q, const int* slots,
                          int num_seqs, int max_tokens, long long total_tokens, float* seg_state, float* seg_decay, float* o,
                          cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(H > 0 && d > 0 && d <= 256 && dv > 0 && tau > 0.f && ld >= 2 * H * d + H * dv,
               "gla_scan: bad sizes H=%d d=%d dv=%d ld=%d (key size at most 256)", H, d, dv, ld);
    const bool cut = seg_state != nullptr && seg_decay != nullptr && max_tokens >= 2 * GLA_SEG;
    const int segs = cut ? (max_tokens + GLA_SEG - 1) / GLA_SEG - 1 : 1;    // blocks per request in each launch
    const dim3 grid((unsigned)num_seqs * segs, H, (dv + GLA_COLS - 1) / GLA_COLS);
    PL_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gla_scan: %d heads of %d values", H, dv);
    const int nper = (d + GLA_LANES - 1) / GLA_LANES;
    const float* zb = z_bias;
    if (cut) {
        const long long n = total_tokens * H * d, blocks = (n + 255) / 256;
        PL_REQUIRE(total_tokens > 0, "gla_scan: %lld tokens", total_tokens);
        gla_decay_kernel<<<(unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16), 256, 0, stream>>>(z, z_bias, H * d, 1.0f / tau, n);
        PL_LAUNCHED("gla_decay");
        zb = nullptr;
    }
#define PL_GLA(TT, N)                                                                                                      \
    gla_scan_kernel<TT, N><<<grid, 128, 0, stream>>>((const TT*)proj, ld, z, zb, H, d, dv, 1.0f / tau, q_scale, state,     \
                                                     state_stride, cu_q, slots, o, cut ? GLA_SEG : 0, segs, second,        \
                                                     seg_state, seg_decay)
#define PL_GLA_N(TT)                                                                                        \
    do {                                                                                                    \
        if (nper <= 2) PL_GLA(TT, 2); else if (nper <= 4) PL_GLA(TT, 4); else if (nper <= 8) PL_GLA(TT, 8); \
        else if (nper <= 16) PL_GLA(TT, 16); else PL_GLA(TT, 32);                                           \
    } while (0)
    for (int second = 0; second < (cut ? 2 : 1); ++second) {
        if (dtype == PL_F32) PL_GLA_N(float);
        else if (dtype == PL_BF16) PL_GLA_N(__nv_bfloat16);
        else return pl_fail("gla_scan: unknown dtype %d", dtype);
        PL_LAUNCHED("gla_scan");
    }
#undef PL_GLA_N
#undef PL_GLA
    return 0;
}

// ------------------------------------------------------------------ gated delta rule
// u: float32 [T, q: G*d | k: G*d | v: H*dv], convolved and activated.  The first kernel makes q and k unit vectors per
// head in place (x / sqrt(sum x^2 + unit_eps); q also times q_scale) and forms, per token and value head,
// beta = sigmoid(b) and g = exp(rate * softplus(a + bias)) from the projection's columns [b: H | a: H] at gate_col0:
// bg[t] = [beta: H | g: H | q . k: G] (the dot of the finished q and k of each q/k head, which the recurrence needs and
// which does not depend on the state).  One warp per (token, q/k head) and one thread per (token, value head).
template <typename T>
__global__ void __launch_bounds__(256) delta_prepare_kernel(float* __restrict__ u, int C, const T* __restrict__ proj, int ld,
                                                            int gate_col0, const float* __restrict__ rate,
                                                            const float* __restrict__ bias, int H, int G, int d,
                                                            float unit_eps, float q_scale, float* __restrict__ bg,
                                                            long long tokens) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BG = 2 * H + G;
    const long long units = tokens * G;                             // (token, q/k head)
    for (long long w = (long long)blockIdx.x * 8 + warp; w < units; w += (long long)gridDim.x * 8) {
        const long long t = w / G;
        const int g = (int)(w - t * G);
        float* q = u + t * C + (size_t)g * d;
        float* k = q + (size_t)G * d;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < d; i += 32) {
            sq = fmaf(q[i], q[i], sq);
            sk = fmaf(k[i], k[i], sk);
        }
        const float rq = (1.0f / sqrtf(warp_sum(sq) + unit_eps)) * q_scale, rk = 1.0f / sqrtf(warp_sum(sk) + unit_eps);
        float dot = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float qv = q[i] * rq, kv = k[i] * rk;
            q[i] = qv;
            k[i] = kv;
            dot = fmaf(qv, kv, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) bg[t * BG + 2 * H + g] = dot;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < tokens * H; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / H;
        const int h = (int)(i - t * H);
        const float b = to_float(proj[t * ld + gate_col0 + h]), a = to_float(proj[t * ld + gate_col0 + H + h]) + __ldg(bias + h);
        const float sp = a > 20.f ? a : log1pf(expf(a));             // softplus
        bg[t * BG + h] = sigmoid_f(b);
        bg[t * BG + H + h] = expf(__ldg(rate + h) * sp);
    }
}

// The recurrence.  grid: (requests, value heads, blocks of COLS = 128 / LANES columns).  A column j of a head's state (the d
// numbers S[:, j]) is independent of the other columns: LANES lanes share it, lane l holding the key channels
// 4 l + 4 LANES m + (0..3), m < NPER / 4, in registers (LANES is 8 unless the caller asks for more).  Per token, with the dots summed over the lanes by a butterfly:
//     a = g (S_j . k),  c = g (S_j . q),  w = beta (v_j - a),  S_j <- g S_j + k w,  o_j = c + (q . k) w
// q, k, v, beta and g of DR_TOK tokens at a time arrive in shared memory by cp.async, the next tokens while these
// are worked on (two buffers).  Each dot runs as four chains whose sums are added in a fixed order, and q . k does not
// wait for the state, so that the chain from token to token is a quarter of a dot, the butterfly and one multiply-add.
// The order of every sum is fixed, so a position's result is bit for bit the same however the prompt was cut and
// whatever else is in the batch.  State of a request, `state_off` floats into its slot: [H][dv][d].
constexpr int DR_THREADS = 128, DR_TOK = 16;

__device__ __forceinline__ void dr_cp4(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(ok ? 4 : 0));
}
__device__ __forceinline__ void dr_cp16(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(ok ? 16 : 0));
}

// Floats of one staging buffer: q and k rows of DP, the block's values, beta, g and q . k (and one row of padding).
__host__ __device__ constexpr int dr_stage_floats(int DP, int COLS) { return DR_TOK * (2 * DP + COLS + 4); }

template <int NPER, int DR_LANES>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(const float* __restrict__ u, int C, const float* __restrict__ bg,
                                                                       int H, int G, int d, int dv, float* __restrict__ state,
                                                                       long long state_stride, long long state_off,
                                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                                       float* __restrict__ out, int vec) {
    constexpr int DP = NPER * DR_LANES;                             // padded key size
    constexpr int THREADS = DR_THREADS, DR_COLS = DR_THREADS / DR_LANES, STAGE = dr_stage_floats(DP, DR_COLS);
    extern __shared__ __align__(16) float dr_smem[];
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    const int tid = threadIdx.x, lane = tid % DR_LANES, col = tid / DR_LANES;
    const int j0 = blockIdx.z * DR_COLS, j = j0 + col;
    const bool live = j < dv;
    const int kvh = h / (H / G);
    float* sp = state + (size_t)slot * state_stride + state_off + ((size_t)h * dv + (live ? j : 0)) * d;
    float S[NPER];
#pragma unroll
    for (int r = 0; r < NPER; ++r) {
        const int ch = (r >> 2) * (4 * DR_LANES) + lane * 4 + (r & 3);
        S[r] = live && ch < d ? sp[ch] : 0.f;
    }
    const float* uq = u + (size_t)q0 * C + (size_t)kvh * d;
    const float* uk = uq + (size_t)G * d;
    const float* uv = u + (size_t)q0 * C + (size_t)2 * G * d + (size_t)h * dv + j0;
    const int BG = 2 * H + G;
    const float* bgp = bg + (size_t)q0 * BG;

    auto stage = [&](int t0, int buf) {
        float* qs = dr_smem + buf * STAGE;
        float* ks = qs + DR_TOK * DP;
        float* vs = ks + DR_TOK * DP;
        float* bs = vs + DR_TOK * DR_COLS;
        const int nt = min(DR_TOK, nq - t0);
        if (vec) {
            for (int e = tid; e < DR_TOK * (DP / 4); e += THREADS) {
                const int tt = e / (DP / 4), ch = (e - tt * (DP / 4)) * 4;
                const bool in = tt < nt && ch < d;
                const size_t off = (size_t)(t0 + (in ? tt : 0)) * C + (in ? ch : 0);
                dr_cp16(qs + tt * DP + ch, uq + off, in);
                dr_cp16(ks + tt * DP + ch, uk + off, in);
            }
        } else {
            for (int e = tid; e < DR_TOK * DP; e += THREADS) {
                const int tt = e / DP, ch = e - tt * DP;
                const bool in = tt < nt && ch < d;
                const size_t off = (size_t)(t0 + (in ? tt : 0)) * C + (in ? ch : 0);
                dr_cp4(qs + e, uq + off, in);
                dr_cp4(ks + e, uk + off, in);
            }
        }
        for (int e = tid; e < DR_TOK * DR_COLS; e += THREADS) {
            const int tt = e / DR_COLS, c = e - tt * DR_COLS;
            const bool in = tt < nt && j0 + c < dv;
            dr_cp4(vs + e, uv + (size_t)(t0 + (in ? tt : 0)) * C + (in ? c : 0), in);
        }
        if (tid < 3 * DR_TOK) {
            const int tt = tid / 3, which = tid - tt * 3;            // beta, g, q . k
            const bool in = tt < nt;
            dr_cp4(bs + which * DR_TOK + tt, bgp + (size_t)(t0 + (in ? tt : 0)) * BG + (which == 2 ? 2 * H + kvh : which * H + h), in);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    stage(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < nq; t0 += DR_TOK, buf ^= 1) {
        const int nt = min(DR_TOK, nq - t0);
        if (t0 + DR_TOK < nq) {
            stage(t0 + DR_TOK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const float* qs = dr_smem + buf * STAGE;
        const float* ks = qs + DR_TOK * DP;
        const float* vs = ks + DR_TOK * DP;
        const float* bs = vs + DR_TOK * DR_COLS;
        const float* gs = bs + DR_TOK;
        const float* es = gs + DR_TOK;
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            float kr[NPER], qr[NPER];
#pragma unroll
            for (int m = 0; m < NPER / 4; ++m) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * DP + m * (4 * DR_LANES) + lane * 4);
                const float4 q4 = *reinterpret_cast<const float4*>(qs + tt * DP + m * (4 * DR_LANES) + lane * 4);
                kr[4 * m] = k4.x, kr[4 * m + 1] = k4.y, kr[4 * m + 2] = k4.z, kr[4 * m + 3] = k4.w;
                qr[4 * m] = q4.x, qr[4 * m + 1] = q4.y, qr[4 * m + 2] = q4.z, qr[4 * m + 3] = q4.w;
            }
            const float g = gs[tt], beta = bs[tt], qk = es[tt], v = vs[tt * DR_COLS + col];
            float a4[4] = {0.f, 0.f, 0.f, 0.f}, c4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < NPER; ++r) {
                a4[r & 3] = fmaf(S[r], kr[r], a4[r & 3]);
                c4[r & 3] = fmaf(S[r], qr[r], c4[r & 3]);
                S[r] *= g;                                          // (off the chain: the decayed state waits for w only)
            }
            float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), c = (c4[0] + c4[1]) + (c4[2] + c4[3]);
            // One butterfly for both sums: after the first step the lower half of a column's lanes carries the partial
            // sums of a, the upper half those of c; a then goes to every lane from the column's first.
            const bool upper = lane >= DR_LANES / 2;
            float x = upper ? c : a;
            x += __shfl_xor_sync(0xffffffffu, upper ? a : c, DR_LANES / 2);
#pragma unroll
            for (int o = DR_LANES / 4; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
            a = __shfl_sync(0xffffffffu, x, (tid & 31) & ~(DR_LANES - 1));
            const float w = beta * (v - g * a);
#pragma unroll
            for (int r = 0; r < NPER; ++r) S[r] = fmaf(kr[r], w, S[r]);
            if (live && lane == DR_LANES / 2) out[(size_t)(q0 + t0 + tt) * H * dv + (size_t)h * dv + j] = fmaf(qk, w, g * x);
        }
        __syncthreads();                                            // the buffer is free for the copies of the chunk after next
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < NPER; ++r) {
            const int ch = (r >> 2) * (4 * DR_LANES) + lane * 4 + (r & 3);
            if (ch < d) sp[ch] = S[r];
        }
    }
}

// out: float32 [T, H*dv].  bg: scratch float32 [T, 2H + G].  u is overwritten (q and k become unit vectors).
PL_EXPORT int pl_delta_rule(float* u, int C, const void* proj, int dtype, int ld, int gate_col0, const float* rate,
                            const float* bias, int H, int G, int d, int dv, float unit_eps, float q_scale, float* bg,
                            float* state, long long state_stride, long long state_off, const int* cu_q, const int* slots,
                            int num_seqs, long long tokens, float* out, int forced_lanes, cudaStream_t stream) {
    if (num_seqs == 0 || tokens == 0) return 0;
    PL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && C == 2 * G * d + H * dv, "delta_rule: bad sizes H=%d G=%d d=%d dv=%d C=%d",
               H, G, d, dv, C);
    PL_REQUIRE(d <= 256, "delta_rule: key size %d above 256", d);
    PL_REQUIRE(gate_col0 >= 0 && gate_col0 + 2 * H <= ld, "delta_rule: gate columns outside the row");
    const long long units = tokens * G;
    const unsigned pb = (unsigned)min((units + 7) / 8 > tokens * H / 256 + 1 ? (units + 7) / 8 : tokens * H / 256 + 1, 8192LL);
    if (dtype == PL_F32)
        delta_prepare_kernel<float><<<pb, 256, 0, stream>>>(u, C, (const float*)proj, ld, gate_col0, rate, bias, H, G, d, unit_eps,
                                                            q_scale, bg, tokens);
    else if (dtype == PL_BF16)
        delta_prepare_kernel<__nv_bfloat16><<<pb, 256, 0, stream>>>(u, C, (const __nv_bfloat16*)proj, ld, gate_col0, rate, bias, H, G,
                                                                    d, unit_eps, q_scale, bg, tokens);
    else
        return pl_fail("delta_rule: unknown dtype %d", dtype);
    PL_LAUNCHED("delta_prepare");
    // 16-byte copies where every row of q and k starts on a 16-byte boundary
    const int vec = d % 4 == 0 && C % 4 == 0 && ((uintptr_t)u & 15) == 0;
#define DELTA_SCAN(N, L)                                                                                                       \
    do {                                                                                                                       \
        constexpr int cols = DR_THREADS / (L);                                                                                 \
        const dim3 grid(num_seqs, H, (dv + cols - 1) / cols);                                                                  \
        PL_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "delta_rule: %d heads of %d values", H, dv);                            \
        const size_t smem = (size_t)2 * dr_stage_floats((N) * (L), cols) * sizeof(float);                                      \
        static bool opted = false;                                                                                             \
        if (!opted && smem > 48 * 1024) {                                                                                      \
            PL_CUDA(cudaFuncSetAttribute(delta_scan_kernel<N, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
            opted = true;                                                                                                      \
        }                                                                                                                      \
        delta_scan_kernel<N, L><<<grid, DR_THREADS, smem, stream>>>(u, C, bg, H, G, d, dv, state, state_stride, state_off,     \
                                                                    cu_q, slots, out, vec);                                    \
    } while (0)
    // Lanes per column: 8 unless the caller asks for 16 or 32.  Measured on one prompt of 2,048 tokens, 16 heads of 128 x 128:
    // 474 us with 8 lanes (16 channels per lane), 501 with 16, 560 with 32 (more warps, but more instructions and
    // shared-memory reads per column); 64 decoding requests 50 / 63 / 87 us.
    const int lanes = forced_lanes == 16 || forced_lanes == 32 ? forced_lanes : 8;
    if (lanes == 8) {
        if (d <= 32) DELTA_SCAN(4, 8);
        else if (d <= 64) DELTA_SCAN(8, 8);
        else if (d <= 128) DELTA_SCAN(16, 8);
        else DELTA_SCAN(32, 8);
    } else if (lanes == 16) {
        if (d <= 64) DELTA_SCAN(4, 16);
        else if (d <= 128) DELTA_SCAN(8, 16);
        else DELTA_SCAN(16, 16);
    } else {
        if (d <= 128) DELTA_SCAN(4, 32);
        else DELTA_SCAN(8, 32);
    }
#undef DELTA_SCAN
    PL_LAUNCHED("delta_scan");
    return 0;
}

// ------------------------------------------------------------------ norm per head, times silu(gate)
// out[t, h*dv + c] = o[t, h, c] / sqrt(mean_c(o[t, h, :]^2) + eps) * w[c] * silu(gate[t, h*dv + c]); one warp per
// (token, head); `gate`: columns of a row-major tensor with row stride ldg.
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ldg,
                                                             const float* __restrict__ w, float eps, T* __restrict__ out,
                                                             long long rows, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= rows * H) return;
    const long long t = item / H;
    const int h = (int)(item - t * H), lane = threadIdx.x & 31;
    const float* orow = o + (size_t)item * dv;
    float sq = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float x = orow[c];
        sq = fmaf(x, x, sq);
    }
    sq = warp_sum(sq);
    const float f = 1.0f / sqrtf(sq / (float)dv + eps);
    const T* g = gate + (size_t)t * ldg + (size_t)h * dv;
    T* dst = out + (size_t)item * dv;
    for (int c = lane; c < dv; c += 32) dst[c] = from_float<T>(orow[c] * f * __ldg(w + c) * silu_f(to_float(g[c])));
}

PL_EXPORT int pl_head_norm_gate(const float* o, const void* gate, int dtype, int ldg, const float* w, float eps, void* out,
                                long long rows, int H, int dv, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && H > 0 && dv > 0, "head_norm_gate: bad sizes rows=%lld H=%d dv=%d", rows, H, dv);
    const long long blocks = (rows * H + 7) / 8;
    PL_REQUIRE(blocks < (1ll << 31), "head_norm_gate: %lld rows", rows);
    if (dtype == PL_F32)
        PL_CUDA(launch_pdl(head_norm_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, o, (const float*)gate, ldg,
                           w, eps, (float*)out, rows, H, dv));
    else if (dtype == PL_BF16)
        PL_CUDA(launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, o,
                           (const __nv_bfloat16*)gate, ldg, w, eps, (__nv_bfloat16*)out, rows, H, dv));
    else
        return pl_fail("head_norm_gate: unknown dtype %d", dtype);
    return 0;
}
