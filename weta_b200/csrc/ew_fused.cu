// A chain of element-wise trait calls as one launch.
//
// The reference issues every unary / binary op of a training step as its own kernel (about 400 launches per step,
// crates/weta-cuda/src/lib.rs:482-521), and a step of the small models is bound by exactly that.  wb_ew_fused runs a
// whole expression of such ops over one index space in a single pass: up to eight strided (or broadcast) f32 inputs
// are read once, a short program of the trait's ops (same codes, same scalar parameters) is interpreted per element
// in registers, and up to four of the intermediate values are stored.  The host layer that builds these programs out
// of an unmodified call stream is weta_b200/fusion.py.
//
// Arithmetic is the stand-alone kernels' (unary.cu, binary.cu): the same expressions, applied in program order, each
// rounded to f32 on its own (-fmad=false), scalar parameters rounded to f32 once.  A fused chain therefore gives
// bit-for-bit what the chain of separate launches gives.
#include "common.h"

namespace {

constexpr int MAX_IN = WB_EWF_MAX_INPUTS, MAX_INSTR = WB_EWF_MAX_INSTRS, MAX_OUT = WB_EWF_MAX_OUTPUTS;

struct Input {
    const float* ptr;
    int nd;          // 0: every element is at ptr[0]; -1: contiguous (element i at ptr[i])
    int32_t size[WB_MAX_DIMS];
    int64_t st[WB_MAX_DIMS];
};

struct Instr {
    int16_t kind, op, a, b;  // kind 0: load input a; 1: unary op on value a; 2: binary op on values a, b
    float p1, p2;
};

struct Program {
    int n_in, n_instr, n_out;
    int64_t n;
    Input in[MAX_IN];
    Instr instr[MAX_INSTR];
    int out_reg[MAX_OUT];
    float* out[MAX_OUT];
};

__device__ __forceinline__ float apply_unary(int op, float v, float p1, float p2) {
    switch (op) {
        case WB_NEG: return -v;
        case WB_EXP: return exp(v);
        case WB_LOG: return log(v);
        case WB_SQRT: return sqrt(v);
        case WB_ABS: return fabs(v);
        case WB_SIGN: return v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f);
        case WB_RELU: return v > 0.f ? v : 0.f;
        case WB_STEP: return v > 0.f ? 1.f : 0.f;
        case WB_TANH: return tanh(v);
        case WB_SIGMOID: {
            if (v >= 0.f) return 1.f / (1.f + exp(-v));
            const float e = exp(v);
            return e / (1.f + e);
        }
        case WB_ERF: return erf(v);
        case WB_SIN: return sin(v);
        case WB_COS: return cos(v);
        case WB_RECIP: return 1.f / v;
        case WB_AFFINE: return v * p1 + p2;
        case WB_POWF: return pow(v, p1);
        case WB_GT_SCALAR: return v > p1 ? 1.f : 0.f;
        case WB_MAX_SCALAR: return (v >= p1 || v != v) ? v : p1;
        default: return (v <= p1 || v != v) ? v : p1;  // WB_MIN_SCALAR
    }
}

__device__ __forceinline__ float apply_binary(int op, float x, float y) {
    switch (op) {
        case WB_ADD: return x + y;
        case WB_SUB: return x - y;
        case WB_MUL: return x * y;
        case WB_DIV: return x / y;
        case WB_POW: return pow(x, y);
        case WB_MAXIMUM: return (x >= y || x != x) ? x : y;
        case WB_MINIMUM: return (x <= y || x != x) ? x : y;
        case WB_EQ: return x == y ? 1.f : 0.f;
        case WB_NE: return x != y ? 1.f : 0.f;
        case WB_LT: return x < y ? 1.f : 0.f;
        case WB_LE: return x <= y ? 1.f : 0.f;
        case WB_GT: return x > y ? 1.f : 0.f;
        default: return x >= y ? 1.f : 0.f;  // WB_GE
    }
}

__global__ void __launch_bounds__(256) ew_fused_kernel(const __grid_constant__ Program p) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < p.n; i += static_cast<int64_t>(gridDim.x) * 256) {
        float v[MAX_INSTR];
#pragma unroll 1
        for (int k = 0; k < p.n_instr; ++k) {
            const Instr& in = p.instr[k];
            if (in.kind == 0) {
                const Input& src = p.in[in.a];
                int64_t off = 0;
                if (src.nd < 0) {
                    off = i;
                } else {
                    int64_t r = i;
                    for (int d = src.nd - 1; d >= 0; --d) {  // row-major decomposition of the shared linear index
                        const int64_t q = r / src.size[d];
                        off += (r - q * src.size[d]) * src.st[d];
                        r = q;
                    }
                }
                v[k] = src.ptr[off];
            } else if (in.kind == 1) {
                v[k] = apply_unary(in.op, v[in.a], in.p1, in.p2);
            } else {
                v[k] = apply_binary(in.op, v[in.a], v[in.b]);
            }
        }
        for (int o = 0; o < p.n_out; ++o) p.out[o][i] = v[p.out_reg[o]];
    }
}

}  // namespace

extern "C" int wb_ew_fused(WbBackend* b, const WbView* inputs, int n_inputs, const WbEwInstr* prog, int n_instr, const int32_t* out_regs,
                           void* const* outs, int n_outputs, int64_t n) {
    WB_REQUIRE(b && prog && out_regs && outs && (inputs || n_inputs == 0), WB_ERR_INVALID, "wb_ew_fused: null pointer");
    WB_REQUIRE(n_inputs >= 0 && n_inputs <= MAX_IN && n_instr > 0 && n_instr <= MAX_INSTR && n_outputs > 0 && n_outputs <= MAX_OUT, WB_ERR_INVALID,
               "wb_ew_fused: %d inputs (<= %d), %d instructions (<= %d), %d outputs (<= %d)", n_inputs, MAX_IN, n_instr, MAX_INSTR, n_outputs,
               MAX_OUT);
    if (n <= 0) return WB_OK;
    Program p{};
    p.n_in = n_inputs;
    p.n_instr = n_instr;
    p.n_out = n_outputs;
    p.n = n;
    for (int i = 0; i < n_inputs; ++i) {
        const WbView& v = inputs[i];
        WB_REQUIRE(v.dtype == WB_F32 && v.data, WB_ERR_UNSUPPORTED, "wb_ew_fused: input %d is not an f32 tensor", i);
        WB_REQUIRE(v.ndim >= 0 && v.ndim <= WB_MAX_DIMS, WB_ERR_INVALID, "wb_ew_fused: input %d has more than 8 dims", i);
        WB_REQUIRE(wb_numel(v) == n, WB_ERR_INVALID, "wb_ew_fused: input %d has %lld elements, the program runs over %lld", i,
                   (long long)wb_numel(v), (long long)n);
        Input& in = p.in[i];
        in.ptr = static_cast<const float*>(v.data) + v.offset;
        if (wb_is_contiguous(v)) {
            in.nd = -1;
            continue;
        }
        // drop size-1 dims; merge neighbours the view steps over exactly
        int nd = 0;
        for (int d = 0; d < v.ndim; ++d) {
            if (v.shape[d] == 1) continue;
            WB_REQUIRE(v.shape[d] < (int64_t(1) << 31), WB_ERR_UNSUPPORTED, "wb_ew_fused: dimension too large");
            if (nd > 0 && in.st[nd - 1] == v.stride[d] * v.shape[d] && static_cast<int64_t>(in.size[nd - 1]) * v.shape[d] < (int64_t(1) << 31)) {
                in.size[nd - 1] = static_cast<int32_t>(in.size[nd - 1] * v.shape[d]);
                in.st[nd - 1] = v.stride[d];
            } else {
                in.size[nd] = static_cast<int32_t>(v.shape[d]);
                in.st[nd] = v.stride[d];
                ++nd;
            }
        }
        in.nd = nd;
    }
    for (int k = 0; k < n_instr; ++k) {
        const WbEwInstr& s = prog[k];
        WB_REQUIRE(s.kind >= 0 && s.kind <= 2, WB_ERR_INVALID, "wb_ew_fused: instruction %d has kind %d", k, s.kind);
        if (s.kind == 0) WB_REQUIRE(s.a >= 0 && s.a < n_inputs, WB_ERR_INVALID, "wb_ew_fused: instruction %d loads input %d", k, s.a);
        if (s.kind == 1) WB_REQUIRE(s.a >= 0 && s.a < k && s.op >= WB_NEG && s.op <= WB_MIN_SCALAR, WB_ERR_INVALID, "wb_ew_fused: bad unary instruction %d", k);
        if (s.kind == 2)
            WB_REQUIRE(s.a >= 0 && s.a < k && s.b >= 0 && s.b < k && s.op >= WB_ADD && s.op <= WB_GE, WB_ERR_INVALID, "wb_ew_fused: bad binary instruction %d", k);
        p.instr[k] = Instr{static_cast<int16_t>(s.kind), static_cast<int16_t>(s.op), static_cast<int16_t>(s.a), static_cast<int16_t>(s.b),
                           static_cast<float>(s.p1), static_cast<float>(s.p2)};
    }
    for (int o = 0; o < n_outputs; ++o) {
        WB_REQUIRE(out_regs[o] >= 0 && out_regs[o] < n_instr && outs[o], WB_ERR_INVALID, "wb_ew_fused: bad output %d", o);
        p.out_reg[o] = out_regs[o];
        p.out[o] = static_cast<float*>(outs[o]);
    }
    WbProfileScope ps(b, "ew_fused");
    const int64_t blocks = std::min<int64_t>((n + 255) / 256, static_cast<int64_t>(b->sm_count) * 16);
    ew_fused_kernel<<<static_cast<unsigned>(blocks), 256, 0, b->stream>>>(p);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
