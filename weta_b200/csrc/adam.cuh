// Adam::step (crates/weta-optim/src/lib.rs:210-239) as one pass over an element; every f32 rounding of the
// reference's 13-call chain is kept (each `mul_scalar` is x*s + 0, `add_scalar(eps)` is x*1 + eps).  Shared by the
// stand-alone optimizer kernel and the data-parallel kernel that sums the replicas' gradients first; both are
// compiled with -fmad=false so no product and sum are contracted.
#pragma once

#include <cmath>

struct AdamK {
    float b1, omb1, b2, omb2, inv_sqrt_bc2, eps, step_size, wd, decay_mul, gscale;
    int first, decoupled, has_wd, scale_grad;
};

inline double wb_powi(double a, int n) {  // f64::powi (compiler-rt __powidf2)
    double r = 1.0;
    while (true) {
        if (n & 1) r *= a;
        n /= 2;
        if (n == 0) break;
        a *= a;
    }
    return r;
}

// Scalars of step t >= 1: computed in f64 and rounded to f32 once, as the reference's kernels receive them
// (crates/weta-cpu/src/lib.rs:167-170).
inline AdamK wb_adam_constants(int64_t t, double lr, double beta1, double beta2, double eps, double weight_decay, int decoupled,
                               double grad_scale) {
    const double bc1 = 1.0 - wb_powi(beta1, static_cast<int>(t)), bc2 = 1.0 - wb_powi(beta2, static_cast<int>(t));
    AdamK k;
    k.b1 = static_cast<float>(beta1);
    k.omb1 = static_cast<float>(1.0 - beta1);
    k.b2 = static_cast<float>(beta2);
    k.omb2 = static_cast<float>(1.0 - beta2);
    k.inv_sqrt_bc2 = static_cast<float>(1.0 / std::sqrt(bc2));
    k.eps = static_cast<float>(eps);
    k.step_size = static_cast<float>(lr / bc1);
    k.wd = static_cast<float>(weight_decay);
    k.decay_mul = static_cast<float>(1.0 - lr * weight_decay);
    k.gscale = static_cast<float>(grad_scale);
    k.first = t == 1;
    k.decoupled = decoupled;
    k.has_wd = weight_decay != 0.0;
    k.scale_grad = grad_scale != 1.0;
    return k;
}

#ifdef __CUDACC__
__device__ __forceinline__ void adam_one(float& th, float g, float& mi, float& vi, const AdamK& k) {
    if (k.scale_grad) g = g * k.gscale;
    if (k.has_wd) {
        if (k.decoupled) th = th * k.decay_mul + 0.f;
        else g = g + (th * k.wd + 0.f);
    }
    float gm = g * k.omb1 + 0.f;
    float gv = (g * g) * k.omb2 + 0.f;
    float mn = k.first ? gm : (mi * k.b1 + 0.f) + gm;
    float vn = k.first ? gv : (vi * k.b2 + 0.f) + gv;
    float den = (sqrtf(vn) * k.inv_sqrt_bc2 + 0.f) * 1.f + k.eps;
    th = th - ((mn / den) * k.step_size + 0.f);
    mi = mn;
    vi = vn;
}
#endif
