// Kernels around the attention kernels for mixers that are not plain grouped-query attention, and the
// dynamic-tanh norm.
//
//  * dynamic tanh: y = tanh(alpha x) w + b, elementwise, with the residual sum fused in front of it
//    and a second dynamic tanh (the norm behind a branch) fused in front of the sum;
//  * a norm over the whole query projection and the whole key projection (all heads at once), the
//    queries laid out for the attention kernel and keys and values written to their page slots, with
//    head sizes padded to the size the cache was made for (keys and values of different sizes);
//  * a sigmoid gate on the heads' outputs;
//  * latent attention: the normed latents, the shared rotated key part and the latent written to the
//    cache as one key/value head; the queries assembled as [absorbed query | rotated part].
//
// Norms, angles, gates and sums are float32 whatever the activations' type is.
#include "common.cuh"

// ------------------------------------------------------------------ dynamic tanh
struct DytParams {
    const float* alpha;     // one scalar on the device
    const float* w;         // [H]
    const float* b;         // [H]
};

// x (float32 stream, may be null) += post(branch); y = pre(x).  Either norm may be absent (alpha null):
// without `post` the branch is added as it is, without `pre` nothing is written to y.  With x null,
// y = pre(branch) (a norm alone, of a tensor that is not the stream).
template <typename TB, typename TY>
__global__ void dyt_kernel(float* __restrict__ x, const TB* __restrict__ branch, DytParams post, DytParams pre,
                           TY* __restrict__ y, long long n, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const float a_post = post.alpha != nullptr ? __ldg(post.alpha) : 0.f;
    const float a_pre = pre.alpha != nullptr ? __ldg(pre.alpha) : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % H);
        float v = 0.f;
        if (branch != nullptr) {
            v = to_float(branch[i]);
            if (post.alpha != nullptr) v = tanhf(a_post * v) * __ldg(post.w + c) + __ldg(post.b + c);
        }
        if (x != nullptr) {
            v += x[i];
            if (branch != nullptr) x[i] = v;
        }
        if (y != nullptr) y[i] = from_float<TY>(tanhf(a_pre * v) * __ldg(pre.w + c) + __ldg(pre.b + c));
    }
}

// The same with four columns per thread: grid (column quads / 256, row groups); a thread keeps the norms' weights
// of its four columns in registers and walks the rows.
template <typename T> struct Quad4;
template <> struct Quad4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

__device__ __forceinline__ float4 dyt4(float4 v, float a, float4 w, float4 b) {
    return make_float4(fmaf(tanhf(a * v.x), w.x, b.x), fmaf(tanhf(a * v.y), w.y, b.y), fmaf(tanhf(a * v.z), w.z, b.z),
                       fmaf(tanhf(a * v.w), w.w, b.w));
}

template <typename TB, typename TY>
__global__ void __launch_bounds__(256) dyt4_kernel(float* __restrict__ x, const TB* __restrict__ branch, DytParams post,
                                                   DytParams pre, TY* __restrict__ y, int rows, int H) {
    pdl_launch_dependents();
    const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (c >= H) return;
    // (the norms' parameters are weights: older than the kernel in front)
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float a_post = post.alpha != nullptr ? __ldg(post.alpha) : 0.f;
    const float a_pre = pre.alpha != nullptr ? __ldg(pre.alpha) : 0.f;
    const float4 w1 = post.alpha != nullptr ? Quad4<float>::load(post.w + c) : zero;
    const float4 b1 = post.alpha != nullptr ? Quad4<float>::load(post.b + c) : zero;
    const float4 w2 = pre.alpha != nullptr ? Quad4<float>::load(pre.w + c) : zero;
    const float4 b2 = pre.alpha != nullptr ? Quad4<float>::load(pre.b + c) : zero;
    pdl_wait();
    for (int r = blockIdx.y; r < rows; r += gridDim.y) {
        const size_t i = (size_t)r * H + c;
        float4 v = zero;
        if (branch != nullptr) {
            v = Quad4<TB>::load(branch + i);
            if (post.alpha != nullptr) v = dyt4(v, a_post, w1, b1);
        }
        if (x != nullptr) {
            const float4 s = Quad4<float>::load(x + i);
            v = make_float4(v.x + s.x, v.y + s.y, v.z + s.z, v.w + s.w);
            if (branch != nullptr) Quad4<float>::store(x + i, v);
        }
        if (y != nullptr) Quad4<TY>::store(y + i, dyt4(v, a_pre, w2, b2));
    }
}

template <typename TB, typename TY>
static int launch_dyt(float* x, const void* branch, DytParams post, DytParams pre, void* y, long long n, int H,
                      cudaStream_t stream) {
    const long long rows = n / H;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (H % 4 == 0 && rows < (1ll << 31) && aligned(x) && aligned(branch) && aligned(y) && aligned(post.w) && aligned(post.b) &&
        aligned(pre.w) && aligned(pre.b)) {
        const int bx = (H / 4 + 255) / 256;
        const long long by = rows < 65535 ? rows : 65535;
        PL_CUDA(launch_pdl(dyt4_kernel<TB, TY>, dim3(bx, (unsigned)by), dim3(256), 0, stream, x, (const TB*)branch, post, pre,
                           (TY*)y, (int)rows, H));
        return 0;
    }
    const long long blocks = (n + 255) / 256;
    PL_CUDA(launch_pdl(dyt_kernel<TB, TY>, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream, x,
                       (const TB*)branch, post, pre, (TY*)y, n, H));
    return 0;
}

PL_EXPORT int pl_dyt(float* x, const void* branch, int branch_dtype, const float* post_alpha, const float* post_w,
                     const float* post_b, const float* pre_alpha, const float* pre_w, const float* pre_b, void* y,
                     int y_dtype, long long rows, int H, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && H > 0, "dyt: bad sizes rows=%lld H=%d", rows, H);
    PL_REQUIRE(x != nullptr || branch != nullptr, "dyt: nothing to normalise");
    PL_REQUIRE(y == nullptr || pre_alpha != nullptr, "dyt: an output without a norm");
    DytParams post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
    const long long n = rows * H;
    if (y == nullptr) pre.alpha = nullptr;
    const bool bf_b = branch != nullptr && branch_dtype == PL_BF16;
    const bool bf_y = y != nullptr && y_dtype == PL_BF16;
    if (bf_b && bf_y) return launch_dyt<__nv_bfloat16, __nv_bfloat16>(x, branch, post, pre, y, n, H, stream);
    if (bf_b) return launch_dyt<__nv_bfloat16, float>(x, branch, post, pre, y, n, H, stream);
    if (bf_y) return launch_dyt<float, __nv_bfloat16>(x, branch, post, pre, y, n, H, stream);
    return launch_dyt<float, float>(x, branch, post, pre, y, n, H, stream);
}

// ------------------------------------------------------------------ page slot of a token
struct SlotArgs {
    const int* positions;
    const int* token_seq;
    const int* block_table;
    int bt_stride, num_pages, ps;
};

// Offset (in elements of a [pages, 2, nkv, ps, D] pool) of the key row of kv head 0 of token t, or -1.
__device__ __forceinline__ long long key_slot(const SlotArgs& a, int t, int s, int pos, int nkv, int D) {
    if (s < 0 || pos < 0) return -1;
    const int page = a.block_table[(size_t)s * a.bt_stride + pos / a.ps];
    if (page < 0 || page >= a.num_pages) return -1;
    return (((long long)page * 2) * nkv * a.ps + pos % a.ps) * D;
}

// A head of n elements turned by the angles of one table row `cs` [rd / 2] of (cos, sin): element e < rd is paired
// with e ^ 1 (interleaved) or with e +- rd / 2 (halves), elements from rd on pass.  `dir` = -1 turns back.
// `elem(i)` gives element i of the head before the turn.
template <typename F>
__device__ __forceinline__ float turned(const float2* cs, int rd, int inter, float dir, int e, F elem) {
    const float self = elem(e);
    if (cs == nullptr || e >= rd) return self;
    const int half = rd >> 1;
    int i, partner;
    bool second;
    if (inter) {
        i = e >> 1, partner = e ^ 1, second = e & 1;
    } else {
        second = e >= half, i = second ? e - half : e, partner = second ? e - half : e + half;
    }
    const float2 t = cs[i];
    const float sn = dir * t.y, other = elem(partner);
    return second ? fmaf(self, t.x, other * sn) : fmaf(self, t.x, -other * sn);
}

// A rotary table and how it pairs the elements of a head.
struct RotTable {
    const float2* table;    // [len, rd / 2] or null: no rotation
    int len, rd, inter;
};

// Four consecutive elements c .. c+3 of a head after the rotation in halves (element i < rd/2 pairs with i + rd/2), for
// rd a multiple of 8 so that a quad lies wholly in one half or behind the rotated part.  `self` and `other` are the quads
// at c and at its partner's place, `cs` the table row.
__device__ __forceinline__ float4 turned_quad(const float2* cs, int rd, int c, float4 self, float4 other) {
    if (cs == nullptr || c >= rd) return self;
    const int half = rd >> 1;
    const bool second = c >= half;
    const float4 t01 = *reinterpret_cast<const float4*>(cs + (second ? c - half : c));
    const float4 t23 = *reinterpret_cast<const float4*>(cs + (second ? c - half : c) + 2);
    const float sg = second ? 1.f : -1.f;
    return make_float4(fmaf(self.x, t01.x, sg * other.x * t01.y), fmaf(self.y, t01.z, sg * other.y * t01.w),
                       fmaf(self.z, t23.x, sg * other.z * t23.y), fmaf(self.w, t23.z, sg * other.w * t23.w));
}

// ------------------------------------------------------------------ norm over whole projections + cache write
// proj row: [q: nh*d | k: nkv*d | v: nkv*dv | ...] (k and v only with has_kv).  One block per token.
//   q' = q / sqrt(mean(q^2) + eps) * qw over all nh*d elements at once, the same for k with kw.
// With a table `rot`, q' and k' are then rotated by the token's position over the table's leading elements of each head.
// With t_every > 0 the query is multiplied by 1 + t_coef * ln(floor((position + 1) / t_every) + 1).
// Q out: [T, nh*D], head h at h*D, columns d..D zero.  K and V go to the page slot, padded to D with zeros.
template <typename T>
__global__ void normed_qkv_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ qw,
                                  const float* __restrict__ kw, float eps, T* __restrict__ q_out, T* __restrict__ kv,
                                  SlotArgs sa, int nh, int nkv, int d, int dv, int D, int has_kv, int write, int vec,
                                  RotTable rot, float t_coef, int t_every) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int s = sa.token_seq[t];
    T* qo = q_out + (size_t)t * nh * D;
    if (s < 0) {                                   // a row that pads the step
        for (int i = threadIdx.x; i < nh * D; i += blockDim.x) qo[i] = from_float<T>(0.f);
        return;
    }
    const T* row = proj + (size_t)t * ld;
    const int nq = nh * d, nk = nkv * d;
    float sq = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const float v = to_float(row[i]);
        sq += v * v;
    }
    const int pos = sa.positions[t];
    float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    if (t_every > 0) rq *= 1.0f + t_coef * logf((float)((max(pos, 0) + 1) / t_every) + 1.0f);
    const float2* cs = rot.table != nullptr && pos >= 0 && pos < rot.len ? rot.table + (size_t)pos * (rot.rd >> 1) : nullptr;
    // the rotation four elements at a time: halves, and a rotated width that quads do not straddle
    const bool rot_vec = vec && cs != nullptr && !rot.inter && rot.rd % 8 == 0;
    auto weighted = [&](const T* src, const float* w, int at) {
        const float4 a = Quad4<T>::load(src + at), g = Quad4<float>::load(w + at);
        return make_float4(a.x * g.x, a.y * g.y, a.z * g.z, a.w * g.w);
    };
    auto partner = [&](int c) { return c >= rot.rd ? c : c >= (rot.rd >> 1) ? c - (rot.rd >> 1) : c + (rot.rd >> 1); };
    if (rot_vec) {
        for (int i = threadIdx.x * 4; i < nh * D; i += blockDim.x * 4) {
            const int h = i / D, c = i - h * D;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < d) {
                v = turned_quad(cs, rot.rd, c, weighted(row, qw, h * d + c), weighted(row, qw, h * d + partner(c)));
                v = make_float4(v.x * rq, v.y * rq, v.z * rq, v.w * rq);
            }
            Quad4<T>::store(qo + i, v);
        }
    } else if (cs != nullptr) {
        for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
            const int h = i / D, c = i - h * D;
            const float v = c < d ? turned(cs, rot.rd, rot.inter, 1.f, c, [&](int e) {
                return to_float(row[h * d + e]) * __ldg(qw + h * d + e);
            }) * rq : 0.f;
            qo[i] = from_float<T>(v);
        }
    } else if (vec) {
        for (int i = threadIdx.x * 4; i < nh * D; i += blockDim.x * 4) {
            const int h = i / D, c = i - h * D;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < d) {
                const float4 a = Quad4<T>::load(row + h * d + c), w = Quad4<float>::load(qw + h * d + c);
                v = make_float4(a.x * rq * w.x, a.y * rq * w.y, a.z * rq * w.z, a.w * rq * w.w);
            }
            Quad4<T>::store(qo + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
            const int h = i / D, c = i - h * D;
            qo[i] = from_float<T>(c < d ? to_float(row[h * d + c]) * rq * __ldg(qw + h * d + c) : 0.f);
        }
    }
    if (!has_kv || !write) return;
    const long long slot = key_slot(sa, t, s, pos, nkv, D);
    float sk = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const float v = to_float(row[nq + i]);
        sk += v * v;
    }
    const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)nk + eps);
    if (slot < 0) return;
    const size_t head_stride = (size_t)sa.ps * D, v_off = (size_t)nkv * sa.ps * D;
    if (rot_vec) {
        for (int i = threadIdx.x * 4; i < nkv * D; i += blockDim.x * 4) {
            const int h = i / D, c = i - h * D;
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (c < d) {
                kk = turned_quad(cs, rot.rd, c, weighted(row + nq, kw, h * d + c), weighted(row + nq, kw, h * d + partner(c)));
                kk = make_float4(kk.x * rk, kk.y * rk, kk.z * rk, kk.w * rk);
            }
            if (c < dv) vv = Quad4<T>::load(row + nq + nk + h * dv + c);
            Quad4<T>::store(kv + slot + h * head_stride + c, kk);
            Quad4<T>::store(kv + slot + v_off + h * head_stride + c, vv);
        }
        return;
    }
    if (cs != nullptr) {
        for (int i = threadIdx.x; i < nkv * D; i += blockDim.x) {
            const int h = i / D, c = i - h * D;
            const float kk = c < d ? turned(cs, rot.rd, rot.inter, 1.f, c, [&](int e) {
                return to_float(row[nq + h * d + e]) * __ldg(kw + h * d + e);
            }) * rk : 0.f;
            const float vv = c < dv ? to_float(row[nq + nk + h * dv + c]) : 0.f;
            kv[slot + h * head_stride + c] = from_float<T>(kk);
            kv[slot + v_off + h * head_stride + c] = from_float<T>(vv);
        }
        return;
    }
    if (vec) {
        for (int i = threadIdx.x * 4; i < nkv * D; i += blockDim.x * 4) {
            const int h = i / D, c = i - h * D;
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (c < d) {
                const float4 a = Quad4<T>::load(row + nq + h * d + c), w = Quad4<float>::load(kw + h * d + c);
                kk = make_float4(a.x * rk * w.x, a.y * rk * w.y, a.z * rk * w.z, a.w * rk * w.w);
            }
            if (c < dv) vv = Quad4<T>::load(row + nq + nk + h * dv + c);
            Quad4<T>::store(kv + slot + h * head_stride + c, kk);
            Quad4<T>::store(kv + slot + v_off + h * head_stride + c, vv);
        }
        return;
    }
    for (int i = threadIdx.x; i < nkv * D; i += blockDim.x) {
        const int h = i / D, c = i - h * D;
        const float kk = c < d ? to_float(row[nq + h * d + c]) * rk * __ldg(kw + h * d + c) : 0.f;
        const float vv = c < dv ? to_float(row[nq + nk + h * dv + c]) : 0.f;
        kv[slot + h * head_stride + c] = from_float<T>(kk);
        kv[slot + v_off + h * head_stride + c] = from_float<T>(vv);
    }
}

PL_EXPORT int pl_normed_qkv_write(const void* proj, int dtype, int T, int ld, const float* qw, const float* kw, float eps,
                                  void* q_out, void* kv, const int* positions, const int* token_seq,
                                  const int* block_table, int bt_stride, int num_pages, int ps, int nh, int nkv, int d,
                                  int dv, int D, int has_kv, int write, const float* rot_table, int rot_len, int rot_rd,
                                  int rot_inter, float t_coef, int t_every, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(nh > 0 && nkv > 0 && d > 0 && dv > 0 && D >= d && D >= dv, "normed_qkv_write: bad head sizes d=%d dv=%d D=%d", d,
               dv, D);
    PL_REQUIRE(rot_table == nullptr || (rot_rd > 0 && rot_rd % 2 == 0 && rot_rd <= d), "normed_qkv_write: %d rotated elements of %d",
               rot_rd, d);
    RotTable rot{(const float2*)rot_table, rot_len, rot_rd, rot_inter};
    SlotArgs sa{positions, token_seq, block_table, bt_stride, num_pages, ps};
    // four elements per step where every head, row and pointer allows it
    const int vec = d % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && ld % 4 == 0 && nh * d % 4 == 0 && nkv * d % 4 == 0 &&
                    (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)kv | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)rot_table) & 15) == 0;
    if (dtype == PL_F32)
        normed_qkv_kernel<float><<<T, 256, 0, stream>>>((const float*)proj, ld, qw, kw, eps, (float*)q_out, (float*)kv, sa,
                                                        nh, nkv, d, dv, D, has_kv, write, vec, rot, t_coef, t_every);
    else if (dtype == PL_BF16)
        normed_qkv_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>((const __nv_bfloat16*)proj, ld, qw, kw, eps,
                                                                (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv, sa, nh, nkv,
                                                                d, dv, D, has_kv, write, vec, rot, t_coef, t_every);
    else
        return pl_fail("normed_qkv_write: unknown dtype %d", dtype);
    PL_LAUNCHED("normed_qkv_write");
    return 0;
}

// ------------------------------------------------------------------ sigmoid gate on the heads' outputs
// out[t, h*dv + c] = o[t, h*D + c] * sigmoid(gate[t, h*dv + c]),  c < dv (the padding of a head is dropped).
// gate null: the copy without the padding.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ o, int D, const T* __restrict__ gate, int ldg, T* __restrict__ out,
                                 long long n, int nh, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = nh * dv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / row;
        const int e = (int)(i - t * row), h = e / dv, c = e - h * dv;
        float v = to_float(o[(size_t)t * nh * D + h * D + c]);
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * ldg + e])));
        out[i] = from_float<T>(v);
    }
}

// The same, four elements per thread: grid (quads of a row / 256, row groups).
template <typename T>
__global__ void __launch_bounds__(256) head_gate4_kernel(const T* __restrict__ o, int D, const T* __restrict__ gate, int ldg,
                                                         T* __restrict__ out, int rows, int nh, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (e >= nh * dv) return;
    const int h = e / dv, c = e - h * dv;
    for (int t = blockIdx.y; t < rows; t += gridDim.y) {
        float4 v = Quad4<T>::load(o + (size_t)t * nh * D + h * D + c);
        if (gate != nullptr) {
            const float4 g = Quad4<T>::load(gate + (size_t)t * ldg + e);
            v = make_float4(v.x / (1.0f + expf(-g.x)), v.y / (1.0f + expf(-g.y)), v.z / (1.0f + expf(-g.z)),
                            v.w / (1.0f + expf(-g.w)));
        }
        Quad4<T>::store(out + (size_t)t * nh * dv + e, v);
    }
}

template <typename T>
static int launch_head_gate(const void* o, int T_, int D, const void* gate, int ldg, void* out, int nh, int dv,
                            cudaStream_t stream) {
    if (dv % 4 == 0 && D % 4 == 0 && ldg % 4 == 0 && (((uintptr_t)o | (uintptr_t)gate | (uintptr_t)out) & 15) == 0) {
        const dim3 grid((nh * dv / 4 + 255) / 256, T_ < 65535 ? T_ : 65535);
        PL_CUDA(launch_pdl(head_gate4_kernel<T>, grid, dim3(256), 0, stream, (const T*)o, D, (const T*)gate, ldg, (T*)out, T_, nh, dv));
        return 0;
    }
    const long long n = (long long)T_ * nh * dv;
    const long long blocks = (n + 255) / 256;
    PL_CUDA(launch_pdl(head_gate_kernel<T>, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream, (const T*)o, D,
                       (const T*)gate, ldg, (T*)out, n, nh, dv));
    return 0;
}

PL_EXPORT int pl_head_gate(const void* o, int dtype, int T, int D, const void* gate, int ldg, void* out, int nh, int dv,
                           cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(nh > 0 && dv > 0 && D >= dv, "head_gate: bad sizes dv=%d D=%d", dv, D);
    if (dtype == PL_F32) return launch_head_gate<float>(o, T, D, gate, ldg, out, nh, dv, stream);
    if (dtype == PL_BF16) return launch_head_gate<__nv_bfloat16>(o, T, D, gate, ldg, out, nh, dv, stream);
    return pl_fail("head_gate: unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ latent attention
// down row: [cq: q_rank | c: kv_rank | kr: rot_dim].  One block per token:
//   cq_out = cq / rms(cq) * qw;  c' = c / rms(c) * cw;  kr' = rotate(kr, position)
//   key slot  [c' | kr' | 0 ..D),  value slot [c' | 0 ..D)   (one kv head)
template <typename T>
__global__ void latent_kv_kernel(const T* __restrict__ down, int ld, const float* __restrict__ qw,
                                 const float* __restrict__ cw, float eps, T* __restrict__ cq_out, T* __restrict__ kv,
                                 SlotArgs sa, RotTable rot, int q_rank, int kv_rank, int rot_dim, int D, int write,
                                 int norm_q) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int s = sa.token_seq[t];
    T* cq = norm_q ? cq_out + (size_t)t * q_rank : nullptr;
    if (s < 0) {
        if (norm_q)
            for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[i] = from_float<T>(0.f);
        return;
    }
    const T* row = down + (size_t)t * ld;
    if (norm_q) {
        // (without a query latent the first q_rank columns are the queries themselves and pass as they are)
        float sq = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_float(row[i]);
            sq += v * v;
        }
        const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[i] = from_float<T>(to_float(row[i]) * rq * __ldg(qw + i));
    }
    if (!write) return;
    float sc = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = to_float(row[q_rank + i]);
        sc += v * v;
    }
    const float rc = 1.0f / sqrtf(block_sum(sc, red) / (float)kv_rank + eps);
    const int pos = sa.positions[t];
    const long long slot = key_slot(sa, t, s, pos, 1, D);
    if (slot < 0) return;
    const float2* cs = rot.table != nullptr && pos < rot.len ? rot.table + (size_t)pos * (rot.rd >> 1) : nullptr;
    const T* kr = row + q_rank + kv_rank;
    const size_t v_off = (size_t)sa.ps * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float kk = 0.f, vv = 0.f;
        if (i < kv_rank) {
            kk = vv = to_float(from_float<T>(to_float(row[q_rank + i]) * rc * __ldg(cw + i)));
        } else if (i < kv_rank + rot_dim) {
            kk = turned(cs, rot.rd, rot.inter, 1.f, i - kv_rank, [&](int e) { return to_float(kr[e]); });
        }
        kv[slot + i] = from_float<T>(kk);
        kv[slot + v_off + i] = from_float<T>(vv);
    }
}

PL_EXPORT int pl_latent_kv_write(const void* down, int dtype, int T, int ld, const float* qw, const float* cw, float eps,
                                 void* cq_out, void* kv, const int* positions, const int* token_seq,
                                 const int* block_table, int bt_stride, int num_pages, int ps, const float* table,
                                 int table_len, int rotary_dims, int rot_inter, int q_rank, int kv_rank, int rot_dim, int D,
                                 int write, int norm_q, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && D >= kv_rank + rot_dim, "latent_kv_write: bad sizes");
    PL_REQUIRE(rotary_dims % 2 == 0 && rotary_dims <= rot_dim, "latent_kv_write: %d rotated dimensions of %d", rotary_dims, rot_dim);
    SlotArgs sa{positions, token_seq, block_table, bt_stride, num_pages, ps};
    RotTable rot{rotary_dims > 0 ? (const float2*)table : nullptr, table_len, rotary_dims, rot_inter};
    if (dtype == PL_F32)
        latent_kv_kernel<float><<<T, 128, 0, stream>>>((const float*)down, ld, qw, cw, eps, (float*)cq_out, (float*)kv, sa,
                                                       rot, q_rank, kv_rank, rot_dim, D, write, norm_q);
    else if (dtype == PL_BF16)
        latent_kv_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)down, ld, qw, cw, eps,
                                                               (__nv_bfloat16*)cq_out, (__nv_bfloat16*)kv, sa,
                                                               rot, q_rank, kv_rank, rot_dim, D, write, norm_q);
    else
        return pl_fail("latent_kv_write: unknown dtype %d", dtype);
    PL_LAUNCHED("latent_kv_write");
    return 0;
}

// Q out [T, nh*D]: head h = [q_abs[t, h, 0..kv_rank) | rotate(q[t, h, d..d+rot_dim)) | 0 ..D).
// q_abs: [T, nh*kv_rank] (the unrotated part of the query multiplied into the key up-projection);
// q: rows of `ldq` elements whose first nh*(d + rot_dim) are the heads.
template <typename T>
__global__ void latent_q_kernel(const T* __restrict__ q_abs, const T* __restrict__ q, T* __restrict__ q_out,
                                const int* __restrict__ positions, const int* __restrict__ token_seq,
                                RotTable rot, int nh, int d, int rot_dim, int kv_rank, int D, int ldq) {
    const int t = blockIdx.x;
    const int s = token_seq[t];
    T* qo = q_out + (size_t)t * nh * D;
    if (s < 0) {
        for (int i = threadIdx.x; i < nh * D; i += blockDim.x) qo[i] = from_float<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const float2* cs = rot.table != nullptr && pos >= 0 && pos < rot.len ? rot.table + (size_t)pos * (rot.rd >> 1) : nullptr;
    const T* qa = q_abs + (size_t)t * nh * kv_rank;
    const T* qr = q + (size_t)t * ldq;
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
        const int h = i / D, c = i - h * D;
        float v = 0.f;
        if (c < kv_rank) {
            v = to_float(qa[h * kv_rank + c]);
        } else if (c < kv_rank + rot_dim) {
            const T* part = qr + h * (d + rot_dim) + d;
            v = turned(cs, rot.rd, rot.inter, 1.f, c - kv_rank, [&](int e) { return to_float(part[e]); });
        }
        qo[i] = from_float<T>(v);
    }
}

PL_EXPORT int pl_latent_q(const void* q_abs, const void* q, int dtype, int T, void* q_out, const int* positions,
                          const int* token_seq, const float* table, int table_len, int rotary_dims, int rot_inter, int nh,
                          int d, int rot_dim, int kv_rank, int D, int ldq, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(nh > 0 && d > 0 && D >= kv_rank + rot_dim && ldq >= nh * (d + rot_dim), "latent_q: bad sizes");
    PL_REQUIRE(rotary_dims % 2 == 0 && rotary_dims <= rot_dim, "latent_q: %d rotated dimensions of %d", rotary_dims, rot_dim);
    RotTable rot{rotary_dims > 0 ? (const float2*)table : nullptr, table_len, rotary_dims, rot_inter};
    if (dtype == PL_F32)
        latent_q_kernel<float><<<T, 256, 0, stream>>>((const float*)q_abs, (const float*)q, (float*)q_out, positions,
                                                      token_seq, rot, nh, d, rot_dim, kv_rank, D, ldq);
    else if (dtype == PL_BF16)
        latent_q_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>((const __nv_bfloat16*)q_abs, (const __nv_bfloat16*)q,
                                                              (__nv_bfloat16*)q_out, positions, token_seq,
                                                              rot, nh, d, rot_dim, kv_rank, D, ldq);
    else
        return pl_fail("latent_q: unknown dtype %d", dtype);
    PL_LAUNCHED("latent_q");
    return 0;
}

// ------------------------------------------------------------------ attention whose values are rotated too
// proj row: [q: nh*d | k: nkv*d | v: nkv*dv | ...] with `bias` (float32, the same layout, may be null) added first.
// q and k are turned by the token's position with the table `qk` (rd_qk elements of each head), v with the table
// `vt` over rd_v elements.  Q out: [T, nh*D], head h at h*D, columns d..D zero; K and V go to the token's page slot,
// padded to D with zeros.  One block per token.

// Blocks of 256 threads per row for kernels that walk a row's elements: one for a step of many rows, up to eight where
// the rows are few and each thread would otherwise make many dependent passes.
static inline unsigned row_blocks(int rows, int elements) {
    if (rows >= 512) return 1;
    const int want = (elements + 255) / 256;
    return (unsigned)(want < 1 ? 1 : want > 8 ? 8 : want);
}

template <typename T>
__global__ void rotated_qkv_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ bias, T* __restrict__ q_out,
                                   T* __restrict__ kv, SlotArgs sa, RotTable qk, RotTable vt, int nh, int nkv, int d, int dv,
                                   int D, int write) {
    const int t = blockIdx.x;
    const int s = sa.token_seq[t];
    T* qo = q_out + (size_t)t * nh * D;
    // (a token's elements are spread over the gridDim.y blocks of its row: few tokens, many blocks)
    const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
    if (s < 0) {                                   // a row that pads the step
        for (int i = first; i < nh * D; i += step) qo[i] = from_float<T>(0.f);
        return;
    }
    const int pos = sa.positions[t];
    const T* row = proj + (size_t)t * ld;
    const float2* cs_qk = qk.table != nullptr && pos >= 0 && pos < qk.len ? qk.table + (size_t)pos * (qk.rd >> 1) : nullptr;
    const float2* cs_v = vt.table != nullptr && pos >= 0 && pos < vt.len ? vt.table + (size_t)pos * (vt.rd >> 1) : nullptr;
    for (int i = first; i < nh * D; i += step) {
        const int h = i / D, c = i - h * D;
        float v = 0.f;
        if (c < d) {
            const int base = h * d;
            v = turned(cs_qk, qk.rd, qk.inter, 1.f, c,
                       [&](int e) { return to_float(row[base + e]) + (bias != nullptr ? __ldg(bias + base + e) : 0.f); });
        }
        qo[i] = from_float<T>(v);
    }
    if (!write) return;
    const long long slot = key_slot(sa, t, s, pos, nkv, D);
    if (slot < 0) return;
    const size_t head_stride = (size_t)sa.ps * D, v_off = (size_t)nkv * sa.ps * D;
    const int k0 = nh * d, v0 = nh * d + nkv * d;
    for (int i = first; i < nkv * D; i += step) {
        const int h = i / D, c = i - h * D;
        float kk = 0.f, vv = 0.f;
        if (c < d) {
            const int base = k0 + h * d;
            kk = turned(cs_qk, qk.rd, qk.inter, 1.f, c,
                        [&](int e) { return to_float(row[base + e]) + (bias != nullptr ? __ldg(bias + base + e) : 0.f); });
        }
        if (c < dv) {
            const int base = v0 + h * dv;
            vv = turned(cs_v, vt.rd, vt.inter, 1.f, c,
                        [&](int e) { return to_float(row[base + e]) + (bias != nullptr ? __ldg(bias + base + e) : 0.f); });
        }
        kv[slot + h * head_stride + c] = from_float<T>(kk);
        kv[slot + v_off + h * head_stride + c] = from_float<T>(vv);
    }
}

PL_EXPORT int pl_rotated_qkv_write(const void* proj, int dtype, int T, int ld, const float* bias, void* q_out, void* kv,
                                   const int* positions, const int* token_seq, const int* block_table, int bt_stride,
                                   int num_pages, int ps, const float* qk_table, int qk_len, int qk_rd, int qk_inter,
                                   const float* v_table, int v_len, int v_rd, int v_inter, int nh, int nkv, int d, int dv,
                                   int D, int write, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(nh > 0 && nkv > 0 && d > 0 && dv > 0 && D >= d && D >= dv, "rotated_qkv_write: bad head sizes d=%d dv=%d D=%d", d,
               dv, D);
    PL_REQUIRE(qk_rd % 2 == 0 && qk_rd <= d && v_rd % 2 == 0 && v_rd <= dv, "rotated_qkv_write: rotation of %d / %d elements of "
               "heads of %d / %d", qk_rd, v_rd, d, dv);
    SlotArgs sa{positions, token_seq, block_table, bt_stride, num_pages, ps};
    RotTable qk{(const float2*)qk_table, qk_len, qk_rd, qk_inter}, vt{(const float2*)v_table, v_len, v_rd, v_inter};
    const dim3 grid(T, row_blocks(T, nh * D));
    if (dtype == PL_F32)
        rotated_qkv_kernel<float><<<grid, 256, 0, stream>>>((const float*)proj, ld, bias, (float*)q_out, (float*)kv, sa, qk, vt, nh,
                                                            nkv, d, dv, D, write);
    else if (dtype == PL_BF16)
        rotated_qkv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)proj, ld, bias, (__nv_bfloat16*)q_out,
                                                                    (__nv_bfloat16*)kv, sa, qk, vt, nh, nkv, d, dv, D, write);
    else
        return pl_fail("rotated_qkv_write: unknown dtype %d", dtype);
    PL_LAUNCHED("rotated_qkv_write");
    return 0;
}

// out[t, h*dv + c] = turn_back(o[t, h*D + ..dv], position of t)[c] * sigmoid(gate[t, h]): each head's output (the
// weighted sum of values that were rotated by their own positions) is turned by minus the query's position, then
// gated by one number per head.  `gate` [T, nh] with row stride ldg, or null.
template <typename T>
__global__ void head_unrotate_gate_kernel(const T* __restrict__ o, int D, const T* __restrict__ gate, int ldg,
                                          const int* __restrict__ positions, const int* __restrict__ token_seq, RotTable vt,
                                          T* __restrict__ out, int nh, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const bool real = token_seq[t] >= 0;
    const float2* cs = real && vt.table != nullptr && pos >= 0 && pos < vt.len ? vt.table + (size_t)pos * (vt.rd >> 1) : nullptr;
    const T* orow = o + (size_t)t * nh * D;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < nh * dv; i += gridDim.y * blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        float v = turned(cs, vt.rd, vt.inter, -1.f, c, [&](int e) { return to_float(orow[h * D + e]); });
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * ldg + h])));
        out[(size_t)t * nh * dv + i] = from_float<T>(v);
    }
}

PL_EXPORT int pl_head_unrotate_gate(const void* o, int dtype, int T, int D, const void* gate, int ldg, const int* positions,
                                    const int* token_seq, const float* v_table, int v_len, int v_rd, int v_inter, void* out,
                                    int nh, int dv, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(nh > 0 && dv > 0 && D >= dv && v_rd % 2 == 0 && v_rd <= dv, "head_unrotate_gate: bad sizes dv=%d D=%d rd=%d", dv, D,
               v_rd);
    RotTable vt{(const float2*)v_table, v_len, v_rd, v_inter};
    if (dtype == PL_F32)
        PL_CUDA(launch_pdl(head_unrotate_gate_kernel<float>, dim3(T, row_blocks(T, nh * dv)), dim3(256), 0, stream, (const float*)o, D, (const float*)gate,
                           ldg, positions, token_seq, vt, (float*)out, nh, dv));
    else if (dtype == PL_BF16)
        PL_CUDA(launch_pdl(head_unrotate_gate_kernel<__nv_bfloat16>, dim3(T, row_blocks(T, nh * dv)), dim3(256), 0, stream, (const __nv_bfloat16*)o, D,
                           (const __nv_bfloat16*)gate, ldg, positions, token_seq, vt, (__nv_bfloat16*)out, nh, dv));
    else
        return pl_fail("head_unrotate_gate: unknown dtype %d", dtype);
    return 0;
}

// ------------------------------------------------------------------ two branches, each normed, then their weighted sum
// v = sa * a / rms(a) * wa + sb * b / rms(b) * wb  (each root mean square over the row, eps inside the root; float32).
// With a stream x (float32 [rows, W], updated in place): x += v, then y = x / rms(x) * nw in y's type, all in this one
// kernel (a block per row; the row's v stays in shared memory between the passes).  Without x: sum_out = v (float32).
template <typename T, typename TW, typename TY>
__global__ void __launch_bounds__(256) normed_pair_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          const float* __restrict__ wa, const float* __restrict__ wb, float sa,
                                                          float sb, float pair_eps, float* __restrict__ x,
                                                          float* __restrict__ sum_out, const TW* __restrict__ nw, float eps,
                                                          TY* __restrict__ y, int W, int vec) {
    extern __shared__ float rowv[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * W;
    if (vec) {
        // W % 4 == 0 and W <= 16 * threads: both rows live in registers, four values per access
        constexpr int IT = 4;
        float4 va[IT], vb[IT];
        float ssa = 0.f, ssb = 0.f;
#pragma unroll
        for (int i = 0; i < IT; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            va[i] = vb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < W) {
                va[i] = Quad4<T>::load(a + base + c);
                vb[i] = Quad4<T>::load(b + base + c);
                ssa += va[i].x * va[i].x + va[i].y * va[i].y + va[i].z * va[i].z + va[i].w * va[i].w;
                ssb += vb[i].x * vb[i].x + vb[i].y * vb[i].y + vb[i].z * vb[i].z + vb[i].w * vb[i].w;
            }
        }
        const float ra = sa / sqrtf(block_sum(ssa, red) / (float)W + pair_eps);
        const float rb = sb / sqrtf(block_sum(ssb, red) / (float)W + pair_eps);
        float ssx = 0.f;
#pragma unroll
        for (int i = 0; i < IT; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            if (c < W) {
                const float4 ga = Quad4<float>::load(wa + c), gb = Quad4<float>::load(wb + c);
                float4 v = make_float4(va[i].x * ra * ga.x + vb[i].x * rb * gb.x, va[i].y * ra * ga.y + vb[i].y * rb * gb.y,
                                       va[i].z * ra * ga.z + vb[i].z * rb * gb.z, va[i].w * ra * ga.w + vb[i].w * rb * gb.w);
                if (x != nullptr) {
                    const float4 xv = Quad4<float>::load(x + base + c);
                    v = make_float4(v.x + xv.x, v.y + xv.y, v.z + xv.z, v.w + xv.w);
                    Quad4<float>::store(x + base + c, v);
                    ssx += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                } else {
                    Quad4<float>::store(sum_out + base + c, v);
                }
                va[i] = v;
            }
        }
        if (x == nullptr) return;
        const float rx = 1.0f / sqrtf(block_sum(ssx, red) / (float)W + eps);
#pragma unroll
        for (int i = 0; i < IT; ++i) {
            const int c = (threadIdx.x + i * 256) * 4;
            if (c < W) {
                const float4 g = Quad4<TW>::load(nw + c);
                Quad4<TY>::store(y + base + c, make_float4(va[i].x * rx * g.x, va[i].y * rx * g.y, va[i].z * rx * g.z, va[i].w * rx * g.w));
            }
        }
        return;
    }
    float ssa = 0.f, ssb = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float va = to_float(a[base + c]), vb = to_float(b[base + c]);
        ssa = fmaf(va, va, ssa);
        ssb = fmaf(vb, vb, ssb);
    }
    const float ra = sa / sqrtf(block_sum(ssa, red) / (float)W + pair_eps);
    const float rb = sb / sqrtf(block_sum(ssb, red) / (float)W + pair_eps);
    float ssx = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = to_float(a[base + c]) * ra * __ldg(wa + c) + to_float(b[base + c]) * rb * __ldg(wb + c);
        if (x != nullptr) {
            v += x[base + c];
            x[base + c] = v;
            rowv[c] = v;
            ssx = fmaf(v, v, ssx);
        } else {
            sum_out[base + c] = v;
        }
    }
    if (x == nullptr) return;
    const float rx = 1.0f / sqrtf(block_sum(ssx, red) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) y[base + c] = from_float<TY>(rowv[c] * rx * to_float(nw[c]));
}

template <typename T, typename TW, typename TY>
static int launch_normed_pair(const void* a, const void* b, const float* wa, const float* wb, float sa, float sb, float pair_eps,
                              float* x, float* sum_out, const void* nw, float eps, void* y, long long rows, int W,
                              cudaStream_t stream) {
    const int vec = W % 4 == 0 && W <= 16 * 256 &&
                    (((uintptr_t)a | (uintptr_t)b | (uintptr_t)wa | (uintptr_t)wb | (uintptr_t)x | (uintptr_t)sum_out | (uintptr_t)nw |
                      (uintptr_t)y) & 15) == 0;
    PL_CUDA(launch_pdl(normed_pair_kernel<T, TW, TY>, dim3((unsigned)rows), dim3(256), x != nullptr && !vec ? (size_t)W * 4 : 0, stream,
                       (const T*)a, (const T*)b, wa, wb, sa, sb, pair_eps, x, sum_out, (const TW*)nw, eps, (TY*)y, W, vec));
    return 0;
}

// dtype: of a and b.  x null: sum_out gets the sum; else x is updated and y (y_dtype) gets its norm with nw (nw_dtype).
PL_EXPORT int pl_normed_pair(const void* a, const void* b, int dtype, const float* wa, const float* wb, float sa, float sb,
                             float pair_eps, float* x, float* sum_out, const void* nw, int nw_dtype, float eps, void* y,
                             int y_dtype, long long rows, int W, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && rows < (1LL << 31) && W > 0 && W <= 12 * 1024, "normed_pair: bad sizes rows=%lld W=%d", rows, W);
    PL_REQUIRE((x != nullptr) == (y != nullptr) && (x != nullptr || sum_out != nullptr), "normed_pair: nowhere to write");
    const int key = (dtype << 2) | (nw_dtype << 1) | y_dtype;
#define PAIR(T, TW, TY) return launch_normed_pair<T, TW, TY>(a, b, wa, wb, sa, sb, pair_eps, x, sum_out, nw, eps, y, rows, W, stream)
    switch (key) {
        case 0: PAIR(float, float, float);
        case 1: PAIR(float, float, __nv_bfloat16);
        case 2: PAIR(float, __nv_bfloat16, float);
        case 3: PAIR(float, __nv_bfloat16, __nv_bfloat16);
        case 4: PAIR(__nv_bfloat16, float, float);
        case 5: PAIR(__nv_bfloat16, float, __nv_bfloat16);
        case 6: PAIR(__nv_bfloat16, __nv_bfloat16, float);
        case 7: PAIR(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    }
#undef PAIR
    return pl_fail("normed_pair: unknown dtypes %d %d %d", dtype, nw_dtype, y_dtype);
}
