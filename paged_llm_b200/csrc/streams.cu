// Several copies of the residual stream (hyper-connections), norms in parts, and a feed-forward activation that is
// a polynomial of unit-norm powers.
//
//  * embedding rows laid out `copies` times side by side;
//  * one kernel per sublayer boundary: the copies take the branch of the sublayer in front in
//    (x_t <- sum_s mix[s, t] x_s + out[t] y, all t from the old x), the input of the next sublayer is formed
//    (u = sum_s in[s] x_s, or the plain sum of the copies) and normed in `groups` equal consecutive parts, each
//    part divided by its own root mean square;
//  * the weighted sum of two branch outputs with their biases, float32;
//  * PolyNorm: a N(z) + b N(z^2) + c N(z^3) + e with N(v) = v / sqrt(mean(v^2) + eps) over the row.
//
// The copies, the sums and the norms are float32 whatever the activations' type is.
#include "common.cuh"

constexpr int MAX_STREAMS = 8;

// ------------------------------------------------------------------ embedding, `copies` times per row
template <typename TW>
__global__ void embedding_copies_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                        int H, int V, float scale, int copies) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool valid = id >= 0 && id < V;
    const TW* row = table + (size_t)(valid ? id : 0) * H;
    float* o = out + (size_t)t * H * copies;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = valid ? to_float(row[c]) * scale : 0.f;
        for (int k = 0; k < copies; ++k) o[(size_t)k * H + c] = v;
    }
}

PL_EXPORT int pl_embedding_copies(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                                  float scale, int copies, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(T > 0 && H > 0 && V > 0 && copies >= 1, "embedding: bad sizes T=%d H=%d V=%d copies=%d", T, H, V, copies);
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == PL_F32)
        PL_CUDA(launch_pdl(embedding_copies_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, out, H,
                           V, scale, copies));
    else if (table_dtype == PL_BF16)
        PL_CUDA(launch_pdl(embedding_copies_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                           (const __nv_bfloat16*)table, ids, out, H, V, scale, copies));
    else
        return pl_fail("embedding: unknown dtype %d", table_dtype);
    return 0;
}

// ------------------------------------------------------------------ stream update + input sum + norm in parts
// One block per row.  x: [rows, S * W] float32, copy s of a row at s * W.
//   branch (may be null): [rows, W]; with `mix` [S, S] (indexed [from, to]) and `outw` [S] the copies become
//     x_t <- sum_s mix[s, t] x_s + outw[t] * branch; without `mix` every copy gets + branch.  Stored back.
//   a second branch (branch2, may be null) is added to the first before that: y = sa * (branch + bias_a) +
//     sb * (branch2 + bias_b) (the two parts of a mixer that runs two mixers side by side); without branch2,
//     y = branch.
//   u = sum_s inw[s] x_s (inw null: the plain sum), kept in shared memory;
//   y_out = u / sqrt(mean_part(u^2) + eps) * w, the mean over each of G equal consecutive parts of W.
// The sums of squares are formed warp by warp in a fixed order, so a row's result does not depend on the batch.
struct StreamNormArgs {
    float* x;
    const void* branch;
    const void* branch2;
    const float* bias_a;
    const float* bias_b;
    float sa, sb;
    const float* mix;
    const float* outw;
    const float* inw;
    const void* w;
    void* y;
    int S, W, G;
    float eps;
};

// VW values in a row at once (VW = 4: one 16-byte or 8-byte access; the pointers are aligned for it)
template <int VW>
__device__ __forceinline__ void load_vals(const float* p, float (&v)[VW]) {
    if (VW == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[VW > 1 ? 1 : 0] = t.y, v[VW > 2 ? 2 : 0] = t.z, v[VW > 3 ? 3 : 0] = t.w;
    } else {
        v[0] = p[0];
    }
}
template <int VW>
__device__ __forceinline__ void load_vals(const __nv_bfloat16* p, float (&v)[VW]) {
    if (VW == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
        v[0] = lo.x, v[VW > 1 ? 1 : 0] = lo.y, v[VW > 2 ? 2 : 0] = hi.x, v[VW > 3 ? 3 : 0] = hi.y;
    } else {
        v[0] = __bfloat162float(p[0]);
    }
}
template <int VW>
__device__ __forceinline__ void store_vals(float* p, const float (&v)[VW]) {
    if (VW == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[VW > 1 ? 1 : 0], v[VW > 2 ? 2 : 0], v[VW > 3 ? 3 : 0]);
    else p[0] = v[0];
}
template <int VW>
__device__ __forceinline__ void store_vals(__nv_bfloat16* p, const float (&v)[VW]) {
    if (VW == 4) {
        uint2 t;
        *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[VW > 1 ? 1 : 0]);
        *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[VW > 2 ? 2 : 0], v[VW > 3 ? 3 : 0]);
        *reinterpret_cast<uint2*>(p) = t;
    } else {
        p[0] = __float2bfloat16(v[0]);
    }
}

// SMAX: the number of copies this build unrolls for (S <= SMAX); VW: values per access.
template <typename TB, typename TW, typename TY, int SMAX, int VW>
__global__ void __launch_bounds__(256) stream_norm_kernel(StreamNormArgs a) {
    extern __shared__ __align__(16) float u_sh[];    // [W] the sublayer's input, [G] the parts' factors, [warps] partial sums
    pdl_launch_dependents();
    const int S = a.S, W = a.W, G = a.G;
    float* fac = u_sh + W;
    float* partial = fac + G;
    float mix[SMAX][SMAX], outw[SMAX], inw[SMAX];
    // (the connections are weights: older than the kernel in front)
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
        outw[s] = a.outw != nullptr && s < S ? __ldg(a.outw + s) : 1.f;
        inw[s] = a.inw != nullptr && s < S ? __ldg(a.inw + s) : 1.f;
#pragma unroll
        for (int t = 0; t < SMAX; ++t)
            mix[s][t] = a.mix != nullptr && s < S && t < S ? __ldg(a.mix + s * S + t) : (s == t ? 1.f : 0.f);
    }
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xr = a.x + r * (size_t)S * W;
    const TB* b1 = a.branch != nullptr ? (const TB*)a.branch + r * W : nullptr;
    const TB* b2 = a.branch2 != nullptr ? (const TB*)a.branch2 + r * W : nullptr;
    for (int c = threadIdx.x * VW; c < W; c += blockDim.x * VW) {
        float xs[SMAX][VW];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s < S) {
                load_vals<VW>(xr + (size_t)s * W + c, xs[s]);
            } else {
#pragma unroll
                for (int e = 0; e < VW; ++e) xs[s][e] = 0.f;
            }
        }
        if (b1 != nullptr) {
            float y[VW];
            load_vals<VW>(b1 + c, y);
            if (b2 != nullptr || a.bias_a != nullptr) {
                float y2[VW];
                if (b2 != nullptr) load_vals<VW>(b2 + c, y2);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    if (a.bias_a != nullptr) y[e] += __ldg(a.bias_a + c + e);
                    y[e] *= a.sa;
                    if (b2 != nullptr) {
                        if (a.bias_b != nullptr) y2[e] += __ldg(a.bias_b + c + e);
                        y[e] = fmaf(a.sb, y2[e], y[e]);
                    }
                }
            }
            float nx[SMAX][VW];
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    float acc = 0.f;
#pragma unroll
                    for (int s = 0; s < SMAX; ++s)
                        if (s < S) acc = fmaf(mix[s][t], xs[s][e], acc);
                    nx[t][e] = fmaf(outw[t], y[e], acc);
                }
            }
#pragma unroll
            for (int t = 0; t < SMAX; ++t)
                if (t < S) {
#pragma unroll
                    for (int e = 0; e < VW; ++e) xs[t][e] = nx[t][e];
                    store_vals<VW>(xr + (size_t)t * W + c, nx[t]);
                }
        }
        float u[VW];
#pragma unroll
        for (int e = 0; e < VW; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) acc = fmaf(inw[s], xs[s][e], acc);
            u[e] = acc;
        }
        store_vals<VW>(u_sh + c, u);
    }
    __syncthreads();
    if (a.y == nullptr) return;
    const int gw = W / G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    // few parts: each is cut into `split` pieces, a warp sums a piece and the pieces are added in order
    const int split = (G < nw && nw % G == 0 && gw % (nw / G) == 0) ? nw / G : 1;
    if (split > 1) {
        const int g = warp / split, piece = gw / split, from = g * gw + (warp - g * split) * piece;
        float sq = 0.f;
        for (int c = lane; c < piece; c += 32) {
            const float v = u_sh[from + c];
            sq = fmaf(v, v, sq);
        }
        sq = warp_sum(sq);
        if (lane == 0) partial[warp] = sq;
        __syncthreads();
        if (threadIdx.x < G) {
            float sum = 0.f;
            for (int k = 0; k < split; ++k) sum += partial[threadIdx.x * split + k];
            fac[threadIdx.x] = 1.0f / sqrtf(sum / (float)gw + a.eps);
        }
    } else {
        for (int g = warp; g < G; g += nw) {
            float sq = 0.f;
            for (int c = lane; c < gw; c += 32) {
                const float v = u_sh[g * gw + c];
                sq = fmaf(v, v, sq);
            }
            sq = warp_sum(sq);
            if (lane == 0) fac[g] = 1.0f / sqrtf(sq / (float)gw + a.eps);
        }
    }
    __syncthreads();
    TY* yr = (TY*)a.y + r * W;
    const TW* w = (const TW*)a.w;
    for (int c = threadIdx.x * VW; c < W; c += blockDim.x * VW) {
        float u[VW], wv[VW];
        load_vals<VW>(u_sh + c, u);
        load_vals<VW>(w + c, wv);
#pragma unroll
        for (int e = 0; e < VW; ++e) u[e] = u[e] * fac[(c + e) / gw] * wv[e];
        store_vals<VW>(yr + c, u);
    }
}

template <typename TB, typename TW, typename TY, int SMAX>
static int stream_norm_v(const StreamNormArgs& a, bool wide, long long rows, size_t smem, cudaStream_t stream) {
    if (wide) {
        if (smem > 48 * 1024)
            PL_CUDA(cudaFuncSetAttribute(stream_norm_kernel<TB, TW, TY, SMAX, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PL_CUDA(launch_pdl(stream_norm_kernel<TB, TW, TY, SMAX, 4>, dim3((unsigned)rows), dim3(256), smem, stream, a));
    } else {
        if (smem > 48 * 1024)
            PL_CUDA(cudaFuncSetAttribute(stream_norm_kernel<TB, TW, TY, SMAX, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PL_CUDA(launch_pdl(stream_norm_kernel<TB, TW, TY, SMAX, 1>, dim3((unsigned)rows), dim3(256), smem, stream, a));
    }
    return 0;
}

template <typename TB, typename TW, typename TY>
static int stream_norm_s(const StreamNormArgs& a, bool wide, long long rows, size_t smem, cudaStream_t stream) {
    if (a.S <= 1) return stream_norm_v<TB, TW, TY, 1>(a, wide, rows, smem, stream);
    if (a.S <= 2) return stream_norm_v<TB, TW, TY, 2>(a, wide, rows, smem, stream);
    if (a.S <= 4) return stream_norm_v<TB, TW, TY, 4>(a, wide, rows, smem, stream);
    return stream_norm_v<TB, TW, TY, MAX_STREAMS>(a, wide, rows, smem, stream);
}

template <typename TB, typename TW>
static int stream_norm_y(const StreamNormArgs& a, int y_dtype, bool wide, long long rows, size_t smem, cudaStream_t stream) {
    if (y_dtype == PL_BF16) return stream_norm_s<TB, TW, __nv_bfloat16>(a, wide, rows, smem, stream);
    return stream_norm_s<TB, TW, float>(a, wide, rows, smem, stream);
}

PL_EXPORT int pl_stream_norm(float* x, const void* branch, const void* branch2, int branch_dtype, const float* bias_a,
                             const float* bias_b, float sa, float sb, const float* mix, const float* outw, const float* inw,
                             const void* w, int w_dtype, void* y, int y_dtype, long long rows, int S, int W, int G, float eps,
                             cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && rows < (1ll << 31) && W > 0 && S >= 1 && S <= MAX_STREAMS, "stream_norm: bad sizes rows=%lld W=%d S=%d",
               rows, W, S);
    PL_REQUIRE(G >= 1 && W % G == 0, "stream_norm: %d values do not divide into %d parts", W, G);
    PL_REQUIRE(branch2 == nullptr || branch != nullptr, "stream_norm: a second branch without a first");
    const size_t smem = ((size_t)W + G + 8) * sizeof(float);
    PL_REQUIRE(smem <= 200 * 1024, "stream_norm: a row of %d values does not fit shared memory", W);
    StreamNormArgs a{x, branch, branch2, bias_a, bias_b, sa, sb, mix, outw, inw, w, y, S, W, G, eps};
    // four values per access where every row of every operand starts on a 16-byte boundary
    const uintptr_t all = (uintptr_t)x | (uintptr_t)branch | (uintptr_t)branch2 | (uintptr_t)w | (uintptr_t)y;
    const bool wide = W % 4 == 0 && all % 16 == 0;
    const bool bf_b = branch != nullptr && branch_dtype == PL_BF16;
    const bool bf_w = w_dtype == PL_BF16;
    if (bf_b && bf_w) return stream_norm_y<__nv_bfloat16, __nv_bfloat16>(a, y_dtype, wide, rows, smem, stream);
    if (bf_b) return stream_norm_y<__nv_bfloat16, float>(a, y_dtype, wide, rows, smem, stream);
    if (bf_w) return stream_norm_y<float, __nv_bfloat16>(a, y_dtype, wide, rows, smem, stream);
    return stream_norm_y<float, float>(a, y_dtype, wide, rows, smem, stream);
}

// ------------------------------------------------------------------ weighted sum of two branch outputs
// out[r, c] = sa * (a[r, c] + bias_a[c]) + sb * (b[r, c] + bias_b[c]), float32 (either bias may be null).
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ bias_a,
                                  const float* __restrict__ bias_b, float sa, float sb, float* __restrict__ out, long long n,
                                  int W) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % W);
        float va = to_float(a[i]), vb = to_float(b[i]);
        if (bias_a != nullptr) va += __ldg(bias_a + c);
        if (bias_b != nullptr) vb += __ldg(bias_b + c);
        out[i] = fmaf(sb, vb, sa * va);
    }
}

PL_EXPORT int pl_scaled_sum(const void* a, const void* b, int dtype, const float* bias_a, const float* bias_b, float sa,
                            float sb, float* out, long long rows, int W, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && W > 0, "scaled_sum: bad sizes rows=%lld W=%d", rows, W);
    const long long n = rows * W, blocks = (n + 255) / 256;
    const dim3 grid((unsigned)(blocks < 8192 ? blocks : 8192));
    if (dtype == PL_F32)
        PL_CUDA(launch_pdl(scaled_sum_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, (const float*)b, bias_a, bias_b,
                           sa, sb, out, n, W));
    else if (dtype == PL_BF16)
        PL_CUDA(launch_pdl(scaled_sum_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)a,
                           (const __nv_bfloat16*)b, bias_a, bias_b, sa, sb, out, n, W));
    else
        return pl_fail("scaled_sum: unknown dtype %d", dtype);
    return 0;
}

// y[r, c] += bias[c] in place (the sum in float32, rounded to y's type).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, long long n, int W) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] = from_float<T>(to_float(y[i]) + __ldg(bias + (int)(i % W)));
}

PL_EXPORT int pl_add_bias(void* y, int dtype, const float* bias, long long rows, int W, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && W > 0, "add_bias: bad sizes rows=%lld W=%d", rows, W);
    const long long n = rows * W, blocks = (n + 255) / 256;
    const dim3 grid((unsigned)(blocks < 8192 ? blocks : 8192));
    if (dtype == PL_F32)
        PL_CUDA(launch_pdl(add_bias_kernel<float>, grid, dim3(256), 0, stream, (float*)y, bias, n, W));
    else if (dtype == PL_BF16)
        PL_CUDA(launch_pdl(add_bias_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)y, bias, n, W));
    else
        return pl_fail("add_bias: unknown dtype %d", dtype);
    return 0;
}

// ------------------------------------------------------------------ PolyNorm
// One block per row of z [rows, F]: out = a z r1 + b z^2 r2 + c z^3 r3 + e with r_k = 1 / sqrt(mean(z^(2k)) + eps).
// The second pass over the row (the polynomial, by Horner's rule) finds it in the caches.

template <typename T, int VW>
__global__ void __launch_bounds__(256) poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps,
                                                        T* __restrict__ out, int F) {
    __shared__ float red[3][8];
    pdl_launch_dependents();
    const float ca = __ldg(coef), cb = __ldg(coef + 1), cc = __ldg(coef + 2), ce = __ldg(coef + 3);
    pdl_wait();
    const T* zr = z + (size_t)blockIdx.x * F;
    T* o = out + (size_t)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int c = threadIdx.x * VW; c < F; c += blockDim.x * VW) {
        float v[VW];
        load_vals<VW>(zr + c, v);
#pragma unroll
        for (int e = 0; e < VW; ++e) {
            const float v2 = v[e] * v[e];
            s2 += v2;
            s4 = fmaf(v2, v2, s4);
            s6 = fmaf(v2 * v2, v2, s6);
        }
    }
    // the three sums over the block at once: warps first, then the warps' parts in order
    s2 = warp_sum(s2), s4 = warp_sum(s4), s6 = warp_sum(s6);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[0][warp] = s2, red[1][warp] = s4, red[2][warp] = s6;
    __syncthreads();
    s2 = s4 = s6 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s2 += red[0][k], s4 += red[1][k], s6 += red[2][k];
    const float inv = 1.0f / (float)F;
    const float r1 = ca / sqrtf(s2 * inv + eps), r2 = cb / sqrtf(s4 * inv + eps), r3 = cc / sqrtf(s6 * inv + eps);
    for (int c = threadIdx.x * VW; c < F; c += blockDim.x * VW) {
        float v[VW];
        load_vals<VW>(zr + c, v);
#pragma unroll
        for (int e = 0; e < VW; ++e) v[e] = fmaf(v[e], fmaf(v[e], fmaf(v[e], r3, r2), r1), ce);
        store_vals<VW>(o + c, v);
    }
}

template <typename T>
static int poly_norm_launch(const T* z, const float* coef, float eps, T* out, long long rows, int F, cudaStream_t stream) {
    // four values per access where every row starts on a 16-byte boundary
    if (F % 4 == 0 && ((uintptr_t)z | (uintptr_t)out) % 16 == 0)
        PL_CUDA(launch_pdl(poly_norm_kernel<T, 4>, dim3((unsigned)rows), dim3(256), 0, stream, z, coef, eps, out, F));
    else
        PL_CUDA(launch_pdl(poly_norm_kernel<T, 1>, dim3((unsigned)rows), dim3(256), 0, stream, z, coef, eps, out, F));
    return 0;
}

PL_EXPORT int pl_poly_norm(const void* z, int dtype, const float* coef, float eps, void* out, long long rows, int F,
                           cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && rows < (1ll << 31) && F > 0, "poly_norm: bad sizes rows=%lld F=%d", rows, F);
    if (dtype == PL_F32) return poly_norm_launch((const float*)z, coef, eps, (float*)out, rows, F, stream);
    if (dtype == PL_BF16)
        return poly_norm_launch((const __nv_bfloat16*)z, coef, eps, (__nv_bfloat16*)out, rows, F, stream);
    else
        return pl_fail("poly_norm: unknown dtype %d", dtype);
    return 0;
}
