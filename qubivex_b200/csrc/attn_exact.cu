// Paged decode attention in the exact operation order of the reference's `attend`
// (crates/qubivex-compute/src/math.rs:142-155), so that f32 results have the reference's
// bits.  Follows `attn_decode.comp` (crates/qubivex-backend-vulkan/shaders/attn_decode.comp:60-175):
//   scores   each position's sequential fma chain over d from +0, times 1 / sqrt(d);
//   softmax  NaN-ignoring maximum (Rust's f32::max), the portable exp (math.rs:50-75),
//            the sum sequential from +0 in position order by one thread, one division each;
//   values   each output dimension's fma chain over positions from +0 in position order.
// One CTA per (query head, token).  Latency bound by design (fixed-order chains); this is
// the correctness anchor that proves block-table addressing, not the fast path.
//
// This file is compiled with -fmad=false, and every operation whose rounding matters is an
// explicit _rn intrinsic, so the compiler can neither fuse nor reorder them.
#include "qvx_common.cuh"

namespace qvx {

__device__ __forceinline__ float exp_portable(float x) {
    if (x != x) return x;
    if (x > 88.72284f) return __uint_as_float(0x7f800000u);
    if (x < -87.33655f) return 0.0f;
    const float shift = 12582912.0f;
    float kf = __fsub_rn(__fadd_rn(__fmul_rn(x, __uint_as_float(0x3fb8aa3bu)), shift), shift);
    float r = __fmaf_rn(-kf, __uint_as_float(0x3f317200u), x);
    r = __fmaf_rn(-kf, __uint_as_float(0x35bfbe8eu), r);
    float p = __uint_as_float(0x39506967u);
    p = __fmaf_rn(p, r, __uint_as_float(0x3ab743ceu));
    p = __fmaf_rn(p, r, __uint_as_float(0x3c088908u));
    p = __fmaf_rn(p, r, __uint_as_float(0x3d2aa9c1u));
    p = __fmaf_rn(p, r, __uint_as_float(0x3e2aaaaau));
    p = __fmaf_rn(p, r, __uint_as_float(0x3f000000u));
    float y = __fadd_rn(__fmaf_rn(p, __fmul_rn(r, r), r), 1.0f);
    int k = __float2int_rz(kf);
    int k1 = k >> 1;
    float v = __fmul_rn(__fmul_rn(y, __uint_as_float((uint32_t)(k1 + 127) << 23)),
                        __uint_as_float((uint32_t)(k - k1 + 127) << 23));
    return v < 1.17549435e-38f ? 0.0f : v;
}

__device__ __forceinline__ float load_kv(const uint8_t* pool, const Layout& L, uint32_t block, uint32_t slot,
                                         uint32_t kv, uint32_t g, uint32_t i) {
    const uint8_t* p = pool + (uint64_t)block * L.block_bytes + in_block_offset(L, slot, kv, g, i);
    if (L.dtype == QVX_F32) return *reinterpret_cast<const float*>(p);
    return widen16(*reinterpret_cast<const uint16_t*>(p), L.dtype);
}

constexpr int EXACT_THREADS = 256;

// Dynamic shared memory: pr[n] scores, then qs[d].
__global__ void __launch_bounds__(EXACT_THREADS)
attn_exact_kernel(Layout L, const uint8_t* __restrict__ pool, const float* __restrict__ q, float* __restrict__ out,
                  const uint32_t* __restrict__ pos, const uint32_t* __restrict__ blocks,
                  const uint32_t* __restrict__ table_at, uint32_t heads, uint32_t n_cap) {
    extern __shared__ float sm[];
    __shared__ float red[EXACT_THREADS];
    __shared__ float stot;
    const uint32_t h = blockIdx.x, t = blockIdx.y, l = threadIdx.x;
    const uint32_t d = L.d, n = pos[t] + 1u, ta = table_at[t];
    const uint32_t g = h / (heads / L.kvh);
    float* pr = sm;
    float* qs = sm + n_cap;
    const size_t qb = ((size_t)t * heads + h) * d;
    for (uint32_t i = l; i < d; i += EXACT_THREADS) qs[i] = q[qb + i];
    __syncthreads();
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)d));
    float m = __uint_as_float(0xff800000u);
    for (uint32_t j = l; j < n; j += EXACT_THREADS) {
        uint32_t block = blocks[ta + j / L.B], slot = j % L.B;
        float acc = 0.0f;
        for (uint32_t i = 0; i < d; i++) acc = __fmaf_rn(qs[i], load_kv(pool, L, block, slot, 0, g, i), acc);
        float v = __fmul_rn(acc, scale);
        pr[j] = v;
        m = fmaxf(m, v);  // the non-NaN operand when one is NaN, as f32::max
    }
    red[l] = m;
    __syncthreads();
    for (uint32_t w = EXACT_THREADS / 2; w > 0; w /= 2) {
        if (l < w) red[l] = fmaxf(red[l], red[l + w]);
        __syncthreads();
    }
    m = red[0];
    for (uint32_t j = l; j < n; j += EXACT_THREADS) pr[j] = exp_portable(__fsub_rn(pr[j], m));
    __syncthreads();
    if (l == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < n; j++) sum = __fadd_rn(sum, pr[j]);
        stot = sum;
    }
    __syncthreads();
    const float sum = stot;
    for (uint32_t j = l; j < n; j += EXACT_THREADS) pr[j] = __fdiv_rn(pr[j], sum);
    __syncthreads();
    for (uint32_t i = l; i < d; i += EXACT_THREADS) {
        float o = 0.0f;
        uint32_t j = 0;
        // Eight value loads issued ahead of their eight dependent fmas.
        for (; j + 8 <= n; j += 8) {
            float v[8];
#pragma unroll
            for (uint32_t k = 0; k < 8; k++) {
                uint32_t jj = j + k;
                v[k] = load_kv(pool, L, blocks[ta + jj / L.B], jj % L.B, 1, g, i);
            }
#pragma unroll
            for (uint32_t k = 0; k < 8; k++) o = __fmaf_rn(pr[j + k], v[k], o);
        }
        for (; j < n; j++) o = __fmaf_rn(pr[j], load_kv(pool, L, blocks[ta + j / L.B], j % L.B, 1, g, i), o);
        out[qb + i] = o;
    }
}

int32_t launch_attn_exact(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          cudaStream_t s) {
    if (t->s == 0) return QVX_OK;
    size_t n_cap = (size_t)t->max_pos + 1;
    size_t smem = (n_cap + t->L.d) * sizeof(float);
    size_t limit = dev->prop.sharedMemPerBlockOptin;
    if (smem + 2048 > limit)
        return fail(dev, QVX_ERR_UNSUPPORTED,
                    "exact-order attention keeps every score in shared memory: %zu positions need %zu bytes, the "
                    "device offers %zu",
                    n_cap, smem, limit);
    cudaError_t e = cudaFuncSetAttribute(attn_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(dev, e, "exact attention shared memory");
    LaunchTimer timer(dev, QVX_K_EXACT, s);
    dim3 grid((unsigned)t->heads, (unsigned)t->s);
    attn_exact_kernel<<<grid, EXACT_THREADS, smem, s>>>(t->L, (const uint8_t*)pool, q, out, t->d_pos, t->d_blocks,
                                                        t->d_table_at, (uint32_t)t->heads, (uint32_t)n_cap);
    return check_cuda(dev, cudaGetLastError(), "exact attention launch");
}

}  // namespace qvx
