// Correctly rounded ln(x) and cos(t) in double, from double-double arithmetic, for the Normal fill of Backend::random
// (crates/weta-core/src/ops.rs:182-186):
//     v = mean + std * sqrt(-2 * ln(u1)) * cos((2 pi) * u2),   u1 = 1 - unit(seed, 2i) in (0, 1], u2 = unit(seed, 2i + 1) in [0, 1)
// The CPU backend evaluates this in f64 with the platform's libm, whose ln and cos are rounded correctly for all but a
// small fraction of arguments; CUDA's are not (1 and 2 ulp).  Evaluating both functions to ~100 bits and rounding
// once gives the correctly rounded double, so the chain above, whose other steps (multiply, sqrt, add) are IEEE
// operations on both machines, yields the CPU's bits wherever the CPU's libm rounds correctly.
//
// Everything here is built from IEEE double add / multiply / divide / fma only, with no table: the same code, compiled
// for the host (contraction off), runs in the CPU-side test that checks it against arbitrary-precision values.
// Ranges: wb_dd_log for x in [2^-53, 1] (any positive normal double works); wb_dd_cos for t in [0, 8).
#pragma once

#include <stdint.h>

#include <cmath>

#if defined(__CUDACC__)
#define WB_HD __host__ __device__ __forceinline__
#else
#define WB_HD inline
#endif

namespace wbdd {

struct dd {
    double hi, lo;
};

WB_HD dd two_sum(double a, double b) {  // a + b exactly
    double s = a + b;
    double bb = s - a;
    double e = (a - (s - bb)) + (b - bb);
    return {s, e};
}
WB_HD dd quick_two_sum(double a, double b) {  // |a| >= |b|
    double s = a + b;
    return {s, b - (s - a)};
}
WB_HD dd two_prod(double a, double b) {  // a * b exactly
    double p = a * b;
    return {p, fma(a, b, -p)};
}
WB_HD dd add(dd a, dd b) {
    dd s = two_sum(a.hi, b.hi);
    dd t = two_sum(a.lo, b.lo);
    s.lo += t.hi;
    s = quick_two_sum(s.hi, s.lo);
    s.lo += t.lo;
    return quick_two_sum(s.hi, s.lo);
}
WB_HD dd add_d(dd a, double b) {
    dd s = two_sum(a.hi, b);
    s.lo += a.lo;
    return quick_two_sum(s.hi, s.lo);
}
WB_HD dd neg(dd a) { return {-a.hi, -a.lo}; }
WB_HD dd mul(dd a, dd b) {
    dd p = two_prod(a.hi, b.hi);
    p.lo += a.hi * b.lo + a.lo * b.hi;
    return quick_two_sum(p.hi, p.lo);
}
WB_HD dd mul_d(dd a, double b) {
    dd p = two_prod(a.hi, b);
    p.lo += a.lo * b;
    return quick_two_sum(p.hi, p.lo);
}
WB_HD dd div(dd a, dd b) {  // a / b to ~104 bits
    double q1 = a.hi / b.hi;
    dd r = add(a, neg(mul_d(b, q1)));
    double q2 = r.hi / b.hi;
    r = add(r, neg(mul_d(b, q2)));
    double q3 = r.hi / b.hi;
    dd q = quick_two_sum(q1, q2);
    return add_d(q, q3);
}
WB_HD dd div_d(dd a, double b) {  // a / b for a double b
    double q1 = a.hi / b;
    dd p = two_prod(q1, b);
    dd r = add(a, neg(p));
    double q2 = r.hi / b;
    p = two_prod(q2, b);
    r = add(r, neg(p));
    double q3 = r.hi / b;
    dd q = quick_two_sum(q1, q2);
    return add_d(q, q3);
}

// ln(x) = e * ln2 + 2 * atanh(s), s = (m - 1) / (m + 1), x = m * 2^e with m in [sqrt(1/2), sqrt(2)); |s| <= 0.1716.
// atanh(s) = s * sum_k z^k / (2k + 1), z = s^2 <= 0.02944: 22 terms reach 2^-110; the terms from k = 11 on are below
// 2^-56 of the sum and are accumulated in plain double.
WB_HD dd log_dd(double x) {
    // exponent and mantissa without libm: x is a positive normal double
    union { double d; uint64_t u; } c;
    c.d = x;
    int e = static_cast<int>((c.u >> 52) & 0x7ff) - 1023;
    c.u = (c.u & 0x000fffffffffffffull) | 0x3ff0000000000000ull;  // m in [1, 2)
    double m = c.d;
    if (m > 1.4142135623730951) { m *= 0.5; e += 1; }
    const double f = m - 1.0;                    // exact
    const dd s = div(dd{f, 0.0}, two_sum(1.0, m));
    const dd z = mul(s, s);
    double tail = 0.0;
    for (int k = 21; k >= 11; --k) tail = tail * z.hi + 1.0 / static_cast<double>(2 * k + 1);
    dd p = {tail, 0.0};
    for (int k = 10; k >= 0; --k) {
        const double n = static_cast<double>(2 * k + 1);
        const double r_hi = 1.0 / n;
        const double r_lo = fma(-r_hi, n, 1.0) / n;  // 1/n = r_hi + r_lo to ~106 bits
        p = add(mul(p, z), dd{r_hi, r_lo});
    }
    dd at = mul(s, p);
    at.hi *= 2.0;
    at.lo *= 2.0;
    // ln 2 to 106 bits
    const dd ln2 = {0.6931471805599453, 2.3190468138462996e-17};
    return add(mul_d(ln2, static_cast<double>(e)), at);
}

WB_HD double log_rn(double x) {
    if (x == 1.0) return 0.0;
    const dd l = log_dd(x);
    return l.hi + l.lo;
}

// sin and cos of a double-double r, |r| <= pi/4 + a little, as nested series:
//   cos r = 1 - z/(1*2) * (1 - z/(3*4) * (1 - z/(5*6) * ...)),  sin r = r * (1 - z/(2*3) * (1 - z/(4*5) * ...)),  z = r^2.
// Fourteen levels reach 2^-110; levels 8 and deeper weigh less than 2^-50 and run in plain double.
WB_HD dd cos_series(dd r) {
    const dd z = mul(r, r);
    double q = 1.0;
    for (int k = 14; k >= 8; --k) q = 1.0 - z.hi * q / static_cast<double>((2 * k - 1) * (2 * k));
    dd p = {q, 0.0};
    for (int k = 7; k >= 1; --k) p = add_d(neg(div_d(mul(z, p), static_cast<double>((2 * k - 1) * (2 * k)))), 1.0);
    return p;
}
WB_HD dd sin_series(dd r) {
    const dd z = mul(r, r);
    double q = 1.0;
    for (int k = 14; k >= 8; --k) q = 1.0 - z.hi * q / static_cast<double>((2 * k) * (2 * k + 1));
    dd p = {q, 0.0};
    for (int k = 7; k >= 1; --k) p = add_d(neg(div_d(mul(z, p), static_cast<double>((2 * k) * (2 * k + 1)))), 1.0);
    return mul(r, p);
}

// cos(t) for a double t in [0, 8): n = nearest multiple of pi/2, r = t - n * pi/2 from a four-part pi/2 whose first
// three parts have 33 significant bits (so n * part is exact for n <= 5 and the first subtraction is exact).
WB_HD double cos_rn(double t) {
    const double P1 = 1.5707963267341256;       // pi/2, leading 33 bits
    const double P2 = 6.077100506303966e-11;    // next 33 bits
    const double P3 = 2.0222662487111665e-21;   // next 33 bits
    const double P4 = 8.4784276603689e-32;      // the rest, full double
    const double P4L = 2.0151106178881e-48;     // and a little more (only its leading bits matter)
    const int n = static_cast<int>(t * 0.6366197723675814 + 0.5);
    dd r;
    if (n == 0) {
        r = {t, 0.0};
    } else {
        const double dn = static_cast<double>(n);
        const double a1 = t - dn * P1;              // exact (Sterbenz)
        r = two_sum(a1, -(dn * P2));                // exact pair
        r = add_d(r, -(dn * P3));
        const dd p4 = two_prod(dn, P4);
        r = add(r, dd{-p4.hi, -(p4.lo + dn * P4L)});
    }
    dd v;
    switch (n & 3) {
        case 0: v = cos_series(r); break;
        case 1: v = neg(sin_series(r)); break;
        case 2: v = neg(cos_series(r)); break;
        default: v = sin_series(r); break;
    }
    return v.hi + v.lo;
}

// Distribution::Normal sample with every step rounded as the CPU backend rounds it.
WB_HD double normal_exact(double mean, double std, double u1, double u2) {
    const double l = log_rn(u1);
    const double a = sqrt(-2.0 * l);
    const double c = cos_rn(6.283185307179586 * u2);
    return mean + (std * a) * c;
}

}  // namespace wbdd
