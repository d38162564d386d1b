// What the reference does between the QKV projections and attention, with its bits
// (crates/qubivex-backend-cpu/src/sim.rs:333-357; the device statement is
// crates/qubivex-backend-vulkan/shaders/attn_prelude.comp:1-176):
//   1. the clip: z.clamp(-c, c) on q, k and v (Rust's clamp: a NaN stays NaN, -0 stays -0);
//   2. the full-width Q and K norms (`math::rms_norm` per token, crates/qubivex-compute/src/math.rs:88-117:
//      the 64-lane sum of squares of crates/qubivex-compute/src/reduce.rs:12-47, then
//      1 / sqrt(ss / n + eps) with a correctly rounded division and square root, then (x * r) * w);
//   3. RoPE on every head of q and k (`math::rope_rotate`, math.rs:159-168: NeoX pairs (i, i + d/2),
//      two products each rounded, then one subtract or add) from the token's table row [cos.., sin..].
// q, k_new and v_new are changed in place; k_new and v_new are what the host cache keeps.  The
// store into the pool (step 4 of the shader) rides in the attention launch (or the append kernel).
//
// One CTA of 64 threads per (part, token), part 0 = q, 1 = k, 2 = v, as the shader's grid: thread l
// is accumulator lane l of the reduction.  Compiled with -fmad=false; every operation whose rounding
// matters is an explicit _rn intrinsic.
#include "qvx_common.cuh"

namespace qvx {

constexpr int PRELUDE_LANES = 64;

struct PreludeArgs {
    float* q; float* k; float* v;
    const float* q_norm; const float* k_norm;  // both or neither
    const float* rope;                         // s x d
    uint32_t heads, kvh, d;
    float eps, clip;
    uint32_t has_clip;
};

__global__ void __launch_bounds__(PRELUDE_LANES) attn_prelude_kernel(PreludeArgs a) {
    __shared__ float acc[PRELUDE_LANES];
    __shared__ float scale;
    const uint32_t part = blockIdx.x, t = blockIdx.y, l = threadIdx.x;
    const uint32_t nh = part == 0 ? a.heads : a.kvh, n = nh * a.d;
    float* row = (part == 0 ? a.q : part == 1 ? a.k : a.v) + (size_t)t * n;
    if (a.has_clip) {
        const float c = a.clip;
        for (uint32_t i = l; i < n; i += PRELUDE_LANES) {
            const float z = row[i];
            row[i] = z < -c ? -c : (z > c ? c : z);  // a NaN fails both tests and stays
        }
    }
    if (part == 2) return;
    const float* w = part == 0 ? a.q_norm : a.k_norm;
    if (w != nullptr) {
        // Lane l takes elements l, l + 64, ... in increasing order: one fused multiply-add each.
        float s = 0.0f;
        for (uint32_t i = l; i < n; i += PRELUDE_LANES) {
            const float x = row[i];  // this thread's own clipped value
            s = __fmaf_rn(x, x, s);
        }
        acc[l] = s;
        __syncthreads();
        // The fixed halving tree: a[i] += a[i + w] for w = 32, 16, 8, 4, then (a0 + a1) + (a2 + a3).
        for (uint32_t wd = PRELUDE_LANES / 2; wd >= 4; wd >>= 1) {
            if (l < wd) acc[l] = __fadd_rn(acc[l], acc[l + wd]);
            __syncthreads();
        }
        if (l == 0) {
            const float ss = __fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3]));
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), a.eps)));
        }
        __syncthreads();
        const float r = scale;
        for (uint32_t i = l; i < n; i += PRELUDE_LANES) row[i] = __fmul_rn(__fmul_rn(row[i], r), w[i]);
    }
    __syncthreads();  // the pairs below cross lanes when d / 2 is not a multiple of 64
    const uint32_t half = a.d / 2;
    const float* cs = a.rope + (size_t)t * a.d;
    for (uint32_t p = l; p < nh * half; p += PRELUDE_LANES) {
        const uint32_t h = p / half, i = p % half;
        float* hd = row + (size_t)h * a.d;
        const float x1 = hd[i], x2 = hd[i + half], c = cs[i], s = cs[half + i];
        hd[i] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
        hd[i + half] = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
    }
}

int32_t launch_attn_prelude(qvx_device* dev, const Layout& L, size_t heads, size_t s, float* q, float* k_new, float* v_new,
                            const qvx_prelude* p, cudaStream_t stream) {
    if (s == 0) return QVX_OK;
    PreludeArgs a;
    a.q = q; a.k = k_new; a.v = v_new;
    a.q_norm = p->q_norm; a.k_norm = p->k_norm; a.rope = p->rope;
    a.heads = (uint32_t)heads; a.kvh = L.kvh; a.d = L.d;
    a.eps = (float)p->eps;  // the reference narrows the epsilon to f32 first (math.rs:103-104)
    a.clip = p->clip; a.has_clip = p->has_clip ? 1u : 0u;
    LaunchTimer timer(dev, QVX_K_PRELUDE, stream);
    attn_prelude_kernel<<<dim3(3, (unsigned)s), PRELUDE_LANES, 0, stream>>>(a);
    return check_cuda(dev, cudaGetLastError(), "attention prelude launch");
}

}  // namespace qvx
