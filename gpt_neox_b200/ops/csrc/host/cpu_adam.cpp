// Vectorised Adam / AdamW on host memory (optimizer-state offload, `optimizer.type: CPUAdam`).
// Plays the role of DeepSpeed's DeepSpeedCPUAdam (AVX C++) used at megatron/training.py:1096 of the
// reference.  OpenMP over chunks; the inner loop is written so the compiler emits AVX2 FMA code
// (-march=x86-64-v3).  Optionally also writes a bf16 copy of the updated weights (for the device).
#include <cmath>
#include <cstdint>
#include <cstring>

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t rounding = 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<uint16_t>((u + rounding) >> 16);
}

extern "C" void neox_cpu_adam_step(float* p, float* m, float* v, const float* g, uint16_t* bf16_out, long long n,
                                   float lr, float beta1, float beta2, float eps, float weight_decay, float bc1,
                                   float bc2, float grad_scale, int adamw) {
    const float step = lr / bc1;
    const float inv_sqrt_bc2 = 1.0f / std::sqrt(bc2);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        float gi = g[i] * grad_scale;
        float pi = p[i];
        if (!adamw && weight_decay != 0.0f) gi += weight_decay * pi;
        const float mi = beta1 * m[i] + (1.0f - beta1) * gi;
        const float vi = beta2 * v[i] + (1.0f - beta2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        const float denom = std::sqrt(vi) * inv_sqrt_bc2 + eps;
        float upd = step * (mi / denom);
        if (adamw && weight_decay != 0.0f) upd += lr * weight_decay * pi;
        pi -= upd;
        p[i] = pi;
        if (bf16_out) bf16_out[i] = f32_to_bf16(pi);
    }
}
