// pybind11 shims: the Python-visible modules of the quantized-GEMM path, with the module and
// function names and the positional argument order of the reference project's bindings
// (cited per function).  This one source is compiled once per module with
//   -DHKB_SHIM_NAME=<module> -DHKB_SHIM_<MODULE>
// Tensors are duck-typed like in the reference (data_ptr / shape are read from the Python
// object; no torch C++ dependency); unlike the reference the shim also reads dtype, device,
// stride and contiguity and validates them.  All work happens behind the C ABI of
// libhkb200.so; a non-zero status becomes a Python RuntimeError carrying hkb_last_error().
#include <pybind11/pybind11.h>

#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/hkb200.h"

namespace py = pybind11;

namespace {

struct TView {
    void* ptr = nullptr;
    std::vector<int64_t> shape;
    std::string dtype;   // "bfloat16", "float8_e4m3fn", "uint8", "float32", ...
    int device = -1;     // CUDA ordinal, -1 = not a CUDA tensor
    int64_t numel = 1;
    bool none = true;
    const char* name = "";
    int64_t dim(int i) const { return shape.at(i < 0 ? shape.size() + i : i); }
    int rank() const { return (int)shape.size(); }
};

[[noreturn]] void fail(const std::string& m) { throw std::runtime_error(m); }

TView view(const py::object& t, const char* name, bool allow_none = false, bool need_contiguous = true) {
    TView v;
    if (t.is_none()) {
        if (!allow_none) fail(std::string(name) + ": tensor is None");
        return v;
    }
    v.none = false;
    v.ptr = reinterpret_cast<void*>(t.attr("data_ptr")().cast<uint64_t>());
    for (auto d : t.attr("shape").cast<py::tuple>()) {
        v.shape.push_back(d.cast<int64_t>());
        v.numel *= v.shape.back();
    }
    if (py::hasattr(t, "dtype")) {
        v.dtype = py::str(t.attr("dtype")).cast<std::string>();
        auto dot = v.dtype.rfind('.');
        if (dot != std::string::npos) v.dtype = v.dtype.substr(dot + 1);
    }
    if (need_contiguous && py::hasattr(t, "is_contiguous") && !t.attr("is_contiguous")().cast<bool>())
        fail(std::string(name) + ": tensor must be contiguous (row-major, inner stride 1)");
    v.name = name;
    if (py::hasattr(t, "device")) {
        py::object dev = t.attr("device");
        if (py::str(dev.attr("type")).cast<std::string>() == "cuda") {
            py::object idx = dev.attr("index");
            v.device = idx.is_none() ? 0 : idx.cast<int>();
        }
    } else {
        v.device = 0;   // duck-typed object without .device: trust the caller, as the reference does
    }
    return v;
}

void want_dtype(const TView& v, const char* name, std::initializer_list<const char*> ok) {
    if (v.dtype.empty()) return;  // duck-typed object without dtype: trust the caller, as the reference does
    std::string list;
    for (const char* d : ok) {
        if (v.dtype == d) return;
        list += std::string(list.empty() ? "" : "/") + d;
    }
    fail(std::string(name) + ": dtype " + v.dtype + " not accepted (want " + list + ")");
}

void same_device(std::initializer_list<const TView*> vs) {
    int dev = -2;
    for (const TView* v : vs) {
        if (v->none) continue;
        if (v->device < 0) fail(std::string(v->name) + ": tensor must live on a CUDA device (there is no CPU path)");
        if (dev == -2) dev = v->device;
        else if (dev != v->device) fail("all tensors must be on the same CUDA device");
    }
}

// RAII: make the tensors' device current (through torch, which owns the CUDA context) and
// fetch torch's current stream on it.
struct Launch {
    py::object guard;
    void* stream = nullptr;
    explicit Launch(int device) {
        if (device < 0) return;
        py::object cuda = py::module_::import("torch").attr("cuda");
        guard = cuda.attr("device")(device);
        guard.attr("__enter__")();
        stream = reinterpret_cast<void*>(cuda.attr("current_stream")(device).attr("cuda_stream").cast<uint64_t>());
    }
    ~Launch() {
        if (guard) guard.attr("__exit__")(py::none(), py::none(), py::none());
    }
};

void check(int rc) {
    if (rc != HKB_OK) fail(std::string(hkb_last_error()) + " [hkb status " + std::to_string(rc) + "]");
}

int mxfp4_mode(const py::object& mode) {
    std::string m;
    if (!mode.is_none()) m = py::str(mode).cast<std::string>();
    else if (const char* e = std::getenv("HKB_MXFP4_MODE")) m = e;
    if (m.empty() || m == "doc" || m == "0") return HKB_MXFP4_MODE_DOC;
    if (m == "kernel" || m == "1") return HKB_MXFP4_MODE_KERNEL;
    fail("unknown MXFP4 mode '" + m + "' (want 'doc' or 'kernel')");
}

// ---- quantizers ----------------------------------------------------------------------------

// per_token_quant_fwd(input, output, scales): kernels/quantization/quant/kernel.cpp:159-171.
// The code type follows output.dtype: float8_e4m3fn / uint8 -> FP8 (amax/448); int8 -> the
// reference's INT8 mode (amax/127).  Any D % 8 == 0 is accepted (the reference: 4 fixed sizes).
[[maybe_unused]] void per_token_quant_fwd(py::object input, py::object output, py::object scales) {
    TView x = view(input, "input"), q = view(output, "output"), s = view(scales, "scales");
    want_dtype(x, "input", {"bfloat16"});
    want_dtype(q, "output", {"float8_e4m3fn", "uint8", "int8"});
    want_dtype(s, "scales", {"float32"});
    if (x.rank() != 2) fail("input must be [M, D]");
    const int64_t M = x.dim(0), D = x.dim(1);
    if (q.numel != M * D) fail("output must have M*D elements");
    if (s.numel != M) fail("scales must have M elements");
    same_device({&x, &q, &s});
    Launch L(x.device);
    if (q.dtype == "int8") check(hkb_quant_int8_per_token(x.ptr, q.ptr, (float*)s.ptr, M, D, D, L.stream));
    else check(hkb_quant_fp8_per_token(x.ptr, q.ptr, (float*)s.ptr, M, D, D, L.stream));
}

// fused_rmsnorm_fp8_quant_fwd(input, weight, output, scales, eps):
// kernels/quantization/fused_fp8_quant/kernel.cpp:262-275.  weight=None -> pure 1x128 quantizer.
[[maybe_unused]] void fused_rmsnorm_fp8_quant_fwd(py::object input, py::object weight, py::object output,
                                                  py::object scales, float eps) {
    TView x = view(input, "input"), w = view(weight, "weight", true), q = view(output, "output"), s = view(scales, "scales");
    want_dtype(x, "input", {"bfloat16"});
    if (!w.none) want_dtype(w, "weight", {"bfloat16"});
    want_dtype(q, "output", {"float8_e4m3fn", "uint8"});
    want_dtype(s, "scales", {"float32"});
    if (x.rank() != 2) fail("input must be [M, D]");
    const int64_t M = x.dim(0), D = x.dim(1);
    if (D % 128 != 0) fail("Unsupported D=" + std::to_string(D) + ": D must be a multiple of 128");
    if (!w.none && w.numel != D) fail("weight must have D elements");
    if (q.numel != M * D) fail("output must have M*D elements");
    if (s.numel != M * (D / 128)) fail("scales must have M*(D/128) elements");
    same_device({&x, &w, &q, &s});
    Launch L(x.device);
    check(hkb_quant_fp8_1x128(x.ptr, w.none ? nullptr : w.ptr, q.ptr, (float*)s.ptr, M, D, eps, L.stream));
}

// Not in the reference: 128x128 block quantizer that produces the weight operand and the
// transposed b_scale [K/128, N/128] the block-scale GEMM consumes.
[[maybe_unused]] void weight_quant_128x128(py::object weight, py::object output, py::object scales) {
    TView w = view(weight, "weight"), q = view(output, "output"), s = view(scales, "scales");
    want_dtype(w, "weight", {"bfloat16"});
    want_dtype(q, "output", {"float8_e4m3fn", "uint8"});
    want_dtype(s, "scales", {"float32"});
    if (w.rank() != 2) fail("weight must be [N, K]");
    const int64_t N = w.dim(0), K = w.dim(1);
    if (q.numel != N * K) fail("output must have N*K elements");
    if (N % 128 || K % 128) fail("N and K must be multiples of 128");
    if (s.numel != (N / 128) * (K / 128)) fail("scales must have (K/128)*(N/128) elements");
    same_device({&w, &q, &s});
    Launch L(w.device);
    check(hkb_quant_fp8_128x128(w.ptr, q.ptr, (float*)s.ptr, N, K, L.stream));
}

// fused_rmsnorm_mxfp4_quant_fwd(input, weight, output, scales, eps):
// kernels/quantization/fused_mxfp4_quant/kernel.cpp:301-314.  weight=None -> pure quantizer.
[[maybe_unused]] void fused_rmsnorm_mxfp4_quant_fwd(py::object input, py::object weight, py::object output,
                                                    py::object scales, float eps, py::object mode) {
    TView x = view(input, "input"), w = view(weight, "weight", true), q = view(output, "output"), s = view(scales, "scales");
    want_dtype(x, "input", {"bfloat16"});
    if (!w.none) want_dtype(w, "weight", {"bfloat16"});
    want_dtype(q, "output", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(s, "scales", {"uint8", "float8_e8m0fnu"});
    if (x.rank() != 2) fail("input must be [M, D]");
    const int64_t M = x.dim(0), D = x.dim(1);
    if (D % 32 != 0) fail("Unsupported D=" + std::to_string(D) + ": D must be a multiple of 32");
    if (!w.none && w.numel != D) fail("weight must have D elements");
    if (q.numel != M * D / 2) fail("output must have M*D/2 bytes");
    if (s.numel != M * (D / 32)) fail("scales must have M*(D/32) bytes");
    same_device({&x, &w, &q, &s});
    const int m = mxfp4_mode(mode);
    Launch L(x.device);
    check(hkb_quant_mxfp4(x.ptr, w.none ? nullptr : w.ptr, q.ptr, s.ptr, M, D, eps, m, L.stream));
}

// Not in the reference: the same quantizer writing its scales (also, or only when scales is None)
// in the layout the MXFP4 GEMM's tensor-core path reads, so that the GEMM needs no re-layout pass.
[[maybe_unused]] void fused_rmsnorm_mxfp4_quant_tc_fwd(py::object input, py::object weight, py::object output,
                                                       py::object scales, py::object sf_tc, float eps, py::object mode) {
    TView x = view(input, "input"), w = view(weight, "weight", true), q = view(output, "output"), s = view(scales, "scales", true),
          tc = view(sf_tc, "sf_tc");
    want_dtype(x, "input", {"bfloat16"});
    if (!w.none) want_dtype(w, "weight", {"bfloat16"});
    want_dtype(q, "output", {"uint8", "float4_e2m1fn_x2"});
    if (!s.none) want_dtype(s, "scales", {"uint8", "float8_e8m0fnu"});
    want_dtype(tc, "sf_tc", {"uint8", "float8_e8m0fnu"});
    if (x.rank() != 2) fail("input must be [M, D]");
    const int64_t M = x.dim(0), D = x.dim(1);
    if (D % 128 != 0) fail("Unsupported D=" + std::to_string(D) + ": D must be a multiple of 128");
    if (!w.none && w.numel != D) fail("weight must have D elements");
    if (q.numel != M * D / 2) fail("output must have M*D/2 bytes");
    if (!s.none && s.numel != M * (D / 32)) fail("scales must have M*(D/32) bytes");
    if (tc.numel < hkb_mxfp4_sf_tc_bytes(1, M, D)) fail("sf_tc must have sf_tc_bytes(1, M, D) bytes");
    same_device({&x, &w, &q, &s, &tc});
    const int m = mxfp4_mode(mode);
    Launch L(x.device);
    check(hkb_quant_mxfp4_tc(x.ptr, w.none ? nullptr : w.ptr, q.ptr, s.none ? nullptr : s.ptr, tc.ptr, M, D, eps, m, L.stream));
}

// ---- GEMMs ---------------------------------------------------------------------------------

struct GemmDims { int64_t batch, M, N, K; };

// A [.., M, Ka], B [.., N, Ka], C [.., M, N]; leading dimensions multiply into the batch
// (the reference pads every tensor to 4-D with leading ones).
GemmDims gemm_dims(const TView& A, const TView& B, const TView& C, int k_per_byte_num, int k_per_byte_den) {
    if (A.rank() < 2 || B.rank() < 2 || C.rank() < 2) fail("A, B, C must have at least 2 dimensions");
    GemmDims d;
    d.M = A.dim(-2);
    d.K = A.dim(-1) * k_per_byte_num / k_per_byte_den;
    d.N = B.dim(-2);
    if (B.dim(-1) != A.dim(-1)) fail("A and B must have the same K extent (both are K-contiguous: A[M,K], B[N,K])");
    d.batch = A.numel / (A.dim(-2) * A.dim(-1));
    if (B.numel / (B.dim(-2) * B.dim(-1)) != d.batch) fail("A and B batch counts differ");
    if (C.dim(-2) != d.M || C.dim(-1) != d.N || C.numel != d.batch * d.M * d.N) fail("C must be [batch, M, N]");
    return d;
}

void fp8_pts(py::object A_, py::object B_, py::object C_, py::object sa_, py::object sb_, py::object bias_) {
    TView A = view(A_, "A"), B = view(B_, "B"), C = view(C_, "C"), sa = view(sa_, "a_scale"), sb = view(sb_, "b_scale"),
          bias = view(bias_, "bias", true);
    want_dtype(A, "A", {"float8_e4m3fn", "uint8"});
    want_dtype(B, "B", {"float8_e4m3fn", "uint8"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(sa, "a_scale", {"float32"});
    want_dtype(sb, "b_scale", {"float32"});
    if (!bias.none) want_dtype(bias, "bias", {"bfloat16"});
    GemmDims d = gemm_dims(A, B, C, 1, 1);
    if (sa.numel != d.batch * d.M) fail("a_scale must have batch*M elements");
    if (sb.numel != d.batch * d.N) fail("b_scale must have batch*N elements");
    if (!bias.none && bias.numel != d.batch * d.N) fail("bias must have batch*N elements");
    same_device({&A, &B, &C, &sa, &sb, &bias});
    Launch L(A.device);
    check(hkb_gemm_fp8_pts(A.ptr, B.ptr, C.ptr, (const float*)sa.ptr, (const float*)sb.ptr,
                           bias.none ? nullptr : bias.ptr, d.batch, d.M, d.N, d.K, L.stream));
}

// gemm_a8w8_per_token_scale_tk.dispatch(A, B, C, a_scale, b_scale):
// kernels/gemm-basic/gemm_a8w8_per_token_scale/kernel.cpp:165-171
[[maybe_unused]] void dispatch_per_token(py::object A, py::object B, py::object C, py::object sa, py::object sb) {
    fp8_pts(A, B, C, sa, sb, py::none());
}
// gemm_a8w8_tk.dispatch(A, B, a_scale, b_scale, C): kernels/gemm-basic/gemm_a8w8/kernel.cpp:171-174
[[maybe_unused]] void dispatch_a8w8(py::object A, py::object B, py::object sa, py::object sb, py::object C) {
    fp8_pts(A, B, C, sa, sb, py::none());
}
// batched_gemm_a8w8_tk.dispatch(A, B, a_scale, b_scale, C, bias):
// kernels/gemm-batched/batched_gemm_a8w8/kernel.cpp:196-202.  bias present -> added.
[[maybe_unused]] void dispatch_batched_a8w8(py::object A, py::object B, py::object sa, py::object sb, py::object C, py::object bias) {
    fp8_pts(A, B, C, sa, sb, bias);
}

// batched_gemm_a8w8_ptgq dispatch(a, b, b_scale, c, bias):
// kernels/gemm-batched/batched_gemm_a8w8_ptgq/kernel.cpp:241-249.  a bf16 [.., M, K] (quantized per row and
// 64-wide K group inside the kernel), b e4m3fn codes [.., N, K], b_scale one float, bias bf16 [.., 1, N] or None.
[[maybe_unused]] void dispatch_ptgq(py::object A_, py::object B_, py::object bs_, py::object C_, py::object bias_) {
    TView A = view(A_, "a"), B = view(B_, "b"), bs = view(bs_, "b_scale"), C = view(C_, "c"), bias = view(bias_, "bias", true);
    want_dtype(A, "a", {"bfloat16"});
    want_dtype(B, "b", {"float8_e4m3fn", "uint8"});
    want_dtype(bs, "b_scale", {"float32"});
    want_dtype(C, "c", {"bfloat16"});
    if (!bias.none) want_dtype(bias, "bias", {"bfloat16"});
    GemmDims d = gemm_dims(A, B, C, 1, 1);
    if (bs.numel != 1) fail("b_scale must hold one float (per-tensor weight scale)");
    if (!bias.none && bias.numel != d.batch * d.N) fail("bias must have batch*N elements");
    same_device({&A, &B, &bs, &C, &bias});
    Launch L(A.device);
    check(hkb_gemm_fp8_ptgq(A.ptr, B.ptr, (const float*)bs.ptr, C.ptr, bias.none ? nullptr : bias.ptr, d.batch, d.M, d.N, d.K, L.stream));
}

// gemm_a8w8_blockscale_tk.dispatch(A, B, C, a_scale, b_scale):
// kernels/gemm-basic/gemm_a8w8_blockscale/kernel.cpp:174-180.
// a_scale [M, K/128]; b_scale [K/128, N/gn], gn = N / b_scale.shape[1] in {1, 128}.
void blockscale(py::object A_, py::object B_, py::object C_, py::object sa_, py::object sb_, py::object ca_, py::object cb_) {
    TView A = view(A_, "A"), B = view(B_, "B"), C = view(C_, "C"), sa = view(sa_, "a_scale"), sb = view(sb_, "b_scale"),
          ca = view(ca_, "c_a", true), cb = view(cb_, "c_b", true);
    want_dtype(A, "A", {"float8_e4m3fn", "uint8"});
    want_dtype(B, "B", {"float8_e4m3fn", "uint8"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(sa, "a_scale", {"float32"});
    want_dtype(sb, "b_scale", {"float32"});
    GemmDims d = gemm_dims(A, B, C, 1, 1);
    if (d.batch != 1) fail("block-scale GEMM takes 2-D operands");
    if (d.K % 128) fail("K must be a multiple of 128");
    const int64_t kb = d.K / 128;
    if (sa.numel != d.M * kb) fail("a_scale must be [M, K/128]");
    if (sb.numel % kb) fail("b_scale must be [K/128, N/gn]");
    const int64_t ncols = sb.numel / kb;
    if (ncols == 0 || d.N % ncols) fail("b_scale must be [K/128, N/gn]");
    const int64_t gn = d.N / ncols;
    if (gn != 1 && gn != 128) fail("b_scale group size along N must be 1 or 128, got " + std::to_string(gn));
    if (ca.none != cb.none) fail("c_a and c_b go together");
    if (!ca.none) {
        want_dtype(ca, "c_a", {"bfloat16"});
        want_dtype(cb, "c_b", {"bfloat16"});
        if (ca.numel != d.M * d.N || cb.numel != d.M * d.N) fail("c_a and c_b must be [M, N]");
    }
    same_device({&A, &B, &C, &sa, &sb, &ca, &cb});
    Launch L(A.device);
    if (ca.none)
        check(hkb_gemm_fp8_blockscale(A.ptr, B.ptr, C.ptr, (const float*)sa.ptr, (const float*)sb.ptr, gn, d.M, d.N, d.K, L.stream));
    else
        check(hkb_gemm_fp8_blockscale_mul_add(A.ptr, B.ptr, C.ptr, (const float*)sa.ptr, (const float*)sb.ptr, gn, ca.ptr, cb.ptr,
                                              d.M, d.N, d.K, L.stream));
}
[[maybe_unused]] void dispatch_blockscale(py::object A, py::object B, py::object C, py::object sa, py::object sb) {
    blockscale(A, B, C, sa, sb, py::none(), py::none());
}
// Not in the reference (it has no multi-GPU code): the block-scale GEMM writing its [M, N] result into
// the same column slab of several row-major matrices of pitch ldc -- this GPU's and, through
// peer-mapped memory, the other GPUs' copies of the assembled output.  dst_ptrs are raw device
// addresses (first element of the slab in each destination), the local one first.
[[maybe_unused]] void dispatch_blockscale_scatter(py::object A_, py::object B_, py::sequence dst_ptrs, int64_t ldc,
                                                  py::object sa_, py::object sb_) {
    TView A = view(A_, "A"), B = view(B_, "B"), sa = view(sa_, "a_scale"), sb = view(sb_, "b_scale");
    want_dtype(A, "A", {"float8_e4m3fn", "uint8"});
    want_dtype(B, "B", {"float8_e4m3fn", "uint8"});
    want_dtype(sa, "a_scale", {"float32"});
    want_dtype(sb, "b_scale", {"float32"});
    if (A.rank() != 2 || B.rank() != 2 || A.dim(1) != B.dim(1)) fail("A [M, K] and B [N, K] must be 2-D with the same K");
    const int64_t M = A.dim(0), K = A.dim(1), N = B.dim(0);
    if (K % 128 || N % 128) fail("K and N must be multiples of 128");
    if (sa.numel != M * (K / 128)) fail("a_scale must be [M, K/128]");
    if (sb.numel != (K / 128) * (N / 128)) fail("b_scale must be [K/128, N/128]");
    std::vector<void*> dst;
    for (auto h : dst_ptrs) dst.push_back(reinterpret_cast<void*>(h.cast<uint64_t>()));
    if (dst.empty() || dst.size() > 8) fail("1 to 8 destinations");
    same_device({&A, &B, &sa, &sb});
    Launch L(A.device);
    check(hkb_gemm_fp8_blockscale_scatter(A.ptr, B.ptr, dst.data(), (int)dst.size(), ldc, (const float*)sa.ptr,
                                          (const float*)sb.ptr, M, N, K, L.stream));
}
// Diagnostic: the block-scale GEMM from the timeline build; `trace` is an int64 / uint64 CUDA tensor of at least
// SMs * 20 * 64 elements that receives the per-K-block clock readings (layout in the C header).
[[maybe_unused]] void dispatch_blockscale_timeline(py::object A_, py::object B_, py::object C_, py::object sa_, py::object sb_,
                                                   py::object trace_) {
    TView A = view(A_, "A"), B = view(B_, "B"), C = view(C_, "C"), sa = view(sa_, "a_scale"), sb = view(sb_, "b_scale");
    TView tr = view(trace_, "trace");
    want_dtype(A, "A", {"float8_e4m3fn", "uint8"});
    want_dtype(B, "B", {"float8_e4m3fn", "uint8"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(sa, "a_scale", {"float32"});
    want_dtype(sb, "b_scale", {"float32"});
    want_dtype(tr, "trace", {"int64", "uint64"});
    if (A.rank() != 2 || B.rank() != 2 || A.dim(1) != B.dim(1)) fail("A [M, K] and B [N, K] must be 2-D with the same K");
    const int64_t M = A.dim(0), K = A.dim(1), N = B.dim(0);
    if (K % 128 || N % 128) fail("K and N must be multiples of 128");
    if (C.numel != M * N) fail("C must be [M, N]");
    if (sa.numel != M * (K / 128)) fail("a_scale must be [M, K/128]");
    if (sb.numel != (K / 128) * (N / 128)) fail("b_scale must be [K/128, N/128]");
    same_device({&A, &B, &C, &sa, &sb, &tr});
    Launch L(A.device);
    check(hkb_debug_gemm_fp8_blockscale_timeline(A.ptr, B.ptr, C.ptr, (const float*)sa.ptr, (const float*)sb.ptr, M, N, K,
                                                 tr.ptr, tr.numel * 8, L.stream));
}
// fused_gemm_a8w8_blockscale_mul_add_tk.dispatch(a, b, c, a_scale, b_scale, c_a, c_b):
// kernels/gemm-fused/fused_gemm_a8w8_blockscale_mul_add/kernel.cpp:184-193.  C = c_a * gemm + c_b.
[[maybe_unused]] void dispatch_blockscale_mul_add(py::object A, py::object B, py::object C, py::object sa, py::object sb,
                                                  py::object ca, py::object cb) {
    if (ca.is_none() || cb.is_none()) fail("c_a and c_b are required");
    blockscale(A, B, C, sa, sb, ca, cb);
}

// gemm_afp4wfp4_tk.dispatch(A, B, C[, a_scales, b_scales]) and the batched twin:
// kernels/gemm-basic/gemm_afp4wfp4/kernel.cpp:154-158, kernels/gemm-batched/batched_gemm_afp4wfp4/kernel.cpp:164-167.
// Operands are the packed form the reference's header comments specify (u8 [.., K/2] codes +
// e8m0 [.., K/32] scales); the 3-argument bf16 "host-dequantized" form is a bf16 GEMM and is rejected.
void mxfp4(py::object A_, py::object B_, py::object C_, py::object sfa_, py::object sfb_, py::object ca_, py::object cb_) {
    if (sfa_.is_none() || sfb_.is_none())
        fail("gemm_afp4wfp4: pass packed e2m1 codes plus a_scales and b_scales (e8m0); "
             "the host-dequantized bf16 form is not supported");
    TView A = view(A_, "A"), B = view(B_, "B"), C = view(C_, "C"), sfa = view(sfa_, "a_scales"), sfb = view(sfb_, "b_scales");
    want_dtype(A, "A", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(B, "B", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(sfa, "a_scales", {"uint8", "float8_e8m0fnu"});
    want_dtype(sfb, "b_scales", {"uint8", "float8_e8m0fnu"});
    GemmDims d = gemm_dims(A, B, C, 2, 1);
    if (sfa.numel != d.batch * d.M * (d.K / 32)) fail("a_scales must be [batch, M, K/32]");
    if (sfb.numel != d.batch * d.N * (d.K / 32)) fail("b_scales must be [batch, N, K/32]");
    TView ca = view(ca_, "c_a", true), cb = view(cb_, "c_b", true);
    if (ca.none != cb.none) fail("c_a and c_b go together");
    if (!ca.none) {
        want_dtype(ca, "c_a", {"bfloat16"});
        want_dtype(cb, "c_b", {"bfloat16"});
        if (d.batch != 1) fail("the multiply-add form takes 2-D operands");
        if (ca.numel != d.M * d.N || cb.numel != d.M * d.N) fail("c_a and c_b must be [M, N]");
    }
    same_device({&A, &B, &C, &sfa, &sfb, &ca, &cb});
    Launch L(A.device);
    if (ca.none)
        check(hkb_gemm_mxfp4(A.ptr, B.ptr, C.ptr, sfa.ptr, sfb.ptr, d.batch, d.M, d.N, d.K, L.stream));
    else
        check(hkb_gemm_mxfp4_mul_add(A.ptr, B.ptr, C.ptr, sfa.ptr, sfb.ptr, ca.ptr, cb.ptr, d.M, d.N, d.K, L.stream));
}
[[maybe_unused]] void dispatch_mxfp4(py::object A, py::object B, py::object C, py::object sfa, py::object sfb) {
    mxfp4(A, B, C, sfa, sfb, py::none(), py::none());
}
// Not in the reference: scale factors already in the tensor-core layout (see include/hkb200.h).
[[maybe_unused]] int64_t mxfp4_sf_tc_bytes(int64_t batch, int64_t rows, int64_t K) { return hkb_mxfp4_sf_tc_bytes(batch, rows, K); }
[[maybe_unused]] void mxfp4_sf_to_tc(py::object sf_, py::object tc_, int64_t K) {
    TView sf = view(sf_, "scales"), tc = view(tc_, "sf_tc");
    want_dtype(sf, "scales", {"uint8", "float8_e8m0fnu"});
    want_dtype(tc, "sf_tc", {"uint8", "float8_e8m0fnu"});
    if (sf.rank() < 2 || K % 128 || sf.dim(-1) != K / 32) fail("scales must be [.., rows, K/32] with K a multiple of 128");
    const int64_t rows = sf.dim(-2), batch = sf.numel / (rows * sf.dim(-1));
    if (tc.numel < hkb_mxfp4_sf_tc_bytes(batch, rows, K)) fail("sf_tc must have sf_tc_bytes(batch, rows, K) bytes");
    same_device({&sf, &tc});
    Launch L(sf.device);
    check(hkb_mxfp4_sf_to_tc(sf.ptr, tc.ptr, batch, rows, K, L.stream));
}
[[maybe_unused]] void dispatch_mxfp4_tc(py::object A_, py::object B_, py::object C_, py::object sfa_, py::object sfb_,
                                        bool a_is_tc, bool b_is_tc) {
    TView A = view(A_, "A"), B = view(B_, "B"), C = view(C_, "C"), sfa = view(sfa_, "a_scales"), sfb = view(sfb_, "b_scales");
    want_dtype(A, "A", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(B, "B", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(sfa, "a_scales", {"uint8", "float8_e8m0fnu"});
    want_dtype(sfb, "b_scales", {"uint8", "float8_e8m0fnu"});
    GemmDims d = gemm_dims(A, B, C, 2, 1);
    if (a_is_tc ? sfa.numel < hkb_mxfp4_sf_tc_bytes(d.batch, d.M, d.K) : sfa.numel != d.batch * d.M * (d.K / 32))
        fail("a_scales must be [batch, M, K/32], or sf_tc_bytes(batch, M, K) bytes in the tensor-core layout");
    if (b_is_tc ? sfb.numel < hkb_mxfp4_sf_tc_bytes(d.batch, d.N, d.K) : sfb.numel != d.batch * d.N * (d.K / 32))
        fail("b_scales must be [batch, N, K/32], or sf_tc_bytes(batch, N, K) bytes in the tensor-core layout");
    same_device({&A, &B, &C, &sfa, &sfb});
    Launch L(A.device);
    check(hkb_gemm_mxfp4_tc(A.ptr, B.ptr, C.ptr, sfa.ptr, a_is_tc ? 1 : 0, sfb.ptr, b_is_tc ? 1 : 0, d.batch, d.M, d.N, d.K, L.stream));
}
// fused_gemm_afp4wfp4_mul_add_tk.dispatch(a, b, c, a_scale, b_scale, c_a, c_b):
// kernels/gemm-fused/fused_gemm_afp4wfp4_mul_add/kernel.cpp:182-191.  Packed e2m1 / e8m0 operands.
[[maybe_unused]] void dispatch_mxfp4_mul_add(py::object A, py::object B, py::object C, py::object sfa, py::object sfb,
                                             py::object ca, py::object cb) {
    if (ca.is_none() || cb.is_none()) fail("c_a and c_b are required");
    mxfp4(A, B, C, sfa, sfb, ca, cb);
}

// Split-cat epilogues: dispatch(a, b, a_scale, b_scale, y, c1, c2), the field order of the reference's
// globals structs (kernels/gemm-fused/fused_gemm_a8w8_blockscale_split_cat/kernel.cpp:34-45,
// fused_gemm_afp4wfp4_split_cat/kernel.cpp:34-45; the reference binds neither to Python).
// y [M, D, S3], c1 [M, D, S1+S3], c2 [M, D, S2]; D, S1, S2, S3 are read from those shapes.
struct SplitDims { int64_t D, S1, S2, S3; };
SplitDims split_dims(const TView& y, const TView& c1, const TView& c2, int64_t M, int64_t N) {
    if (y.rank() != 3 || c1.rank() != 3 || c2.rank() != 3) fail("y, c1, c2 must be [M, D, S]");
    SplitDims d{c2.dim(1), c1.dim(2) - y.dim(2), c2.dim(2), y.dim(2)};
    if (y.dim(0) != M || c1.dim(0) != M || c2.dim(0) != M || y.dim(1) != d.D || c1.dim(1) != d.D) fail("y, c1, c2 must agree on M and D");
    if (d.S1 <= 0 || d.D * (d.S1 + d.S2) != N) fail("N must equal D * (S1 + S2)");
    return d;
}
[[maybe_unused]] void dispatch_blockscale_split_cat(py::object A_, py::object B_, py::object sa_, py::object sb_, py::object y_,
                                                    py::object c1_, py::object c2_) {
    TView A = view(A_, "a"), B = view(B_, "b"), sa = view(sa_, "a_scale"), sb = view(sb_, "b_scale"), y = view(y_, "y"),
          c1 = view(c1_, "c1"), c2 = view(c2_, "c2");
    want_dtype(A, "a", {"float8_e4m3fn", "uint8"});
    want_dtype(B, "b", {"float8_e4m3fn", "uint8"});
    want_dtype(sa, "a_scale", {"float32"});
    want_dtype(sb, "b_scale", {"float32"});
    for (const TView* t : {&y, &c1, &c2}) want_dtype(*t, t->name, {"bfloat16"});
    if (A.rank() != 2 || B.rank() != 2 || A.dim(1) != B.dim(1)) fail("a [M, K] and b [N, K] must be 2-D with the same K");
    const int64_t M = A.dim(0), K = A.dim(1), N = B.dim(0);
    if (K % 128) fail("K must be a multiple of 128");
    const SplitDims d = split_dims(y, c1, c2, M, N);
    const int64_t kb = K / 128;
    if (sa.numel != M * kb) fail("a_scale must be [M, K/128]");
    if (sb.numel != kb * N && sb.numel * 128 != kb * N) fail("b_scale must be [K/128, N] or [K/128, N/128]");
    const int64_t gn = sb.numel == kb * N ? 1 : 128;
    same_device({&A, &B, &sa, &sb, &y, &c1, &c2});
    Launch L(A.device);
    check(hkb_gemm_fp8_blockscale_split_cat(A.ptr, B.ptr, (const float*)sa.ptr, (const float*)sb.ptr, gn, y.ptr, c1.ptr, c2.ptr,
                                            M, N, K, d.S1, d.S2, d.S3, L.stream));
}
[[maybe_unused]] void dispatch_mxfp4_split_cat(py::object A_, py::object B_, py::object sfa_, py::object sfb_, py::object y_,
                                               py::object c1_, py::object c2_) {
    TView A = view(A_, "a"), B = view(B_, "b"), sfa = view(sfa_, "a_scale"), sfb = view(sfb_, "b_scale"), y = view(y_, "y"),
          c1 = view(c1_, "c1"), c2 = view(c2_, "c2");
    want_dtype(A, "a", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(B, "b", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(sfa, "a_scale", {"uint8", "float8_e8m0fnu"});
    want_dtype(sfb, "b_scale", {"uint8", "float8_e8m0fnu"});
    for (const TView* t : {&y, &c1, &c2}) want_dtype(*t, t->name, {"bfloat16"});
    if (A.rank() != 2 || B.rank() != 2 || A.dim(1) != B.dim(1)) fail("a [M, K/2] and b [N, K/2] must be 2-D with the same K");
    const int64_t M = A.dim(0), K = A.dim(1) * 2, N = B.dim(0);
    const SplitDims d = split_dims(y, c1, c2, M, N);
    if (sfa.numel != M * (K / 32) || sfb.numel != N * (K / 32)) fail("a_scale / b_scale must be [rows, K/32]");
    same_device({&A, &B, &sfa, &sfb, &y, &c1, &c2});
    Launch L(A.device);
    check(hkb_gemm_mxfp4_split_cat(A.ptr, B.ptr, sfa.ptr, sfb.ptr, y.ptr, c1.ptr, c2.ptr, M, N, K, d.S1, d.S2, d.S3, L.stream));
}

// moe_op_gemm_a8w8_blockscale_tk.moe_a8w8_blockscale(...): kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/kernel.cpp:201-246
// and :248-282 -- same name, argument names and order, the stride arguments included.  The strides are
// checked, not used: activations and outputs row-major, weights K-contiguous per output column
// (W viewed as [E, K, N] with stride_wk == 1, i.e. stored [E, N, K] like every other GEMM operand here).
[[maybe_unused]] void moe_a8w8_blockscale(py::object X_, py::object W_, py::object Y_, py::object Xs_, py::object Ws_, py::object bias_,
                                          py::object gather_, py::object hist_, py::object offs_, py::object data_,
                                          int64_t N, int64_t K, int64_t group_k, int64_t group_n, int64_t grid_m, int64_t grid_n,
                                          int64_t n_expts_act, int64_t stride_ym, int64_t stride_yn, int64_t stride_xm, int64_t stride_xk,
                                          int64_t stride_we, int64_t stride_wk, int64_t stride_wn, int64_t stride_xsm, int64_t stride_xsk,
                                          int64_t stride_wse, int64_t stride_wsk, int64_t stride_wsn) {
    (void)grid_n;       // the tile width is chosen here
    // W is the one tensor that may arrive as a non-contiguous view ([E, K, N] over [E, N, K] storage)
    TView W = view(W_, "W", false, false);
    TView X = view(X_, "X"), Y = view(Y_, "Y"), Xs = view(Xs_, "X_scale"), Ws = view(Ws_, "W_scale"), bias = view(bias_, "bias", true),
          gather = view(gather_, "GatherIndx", true), hist = view(hist_, "ExptHist"), offs = view(offs_, "ExptOffs"), data = view(data_, "ExptData");
    want_dtype(X, "X", {"float8_e4m3fn", "uint8"});
    want_dtype(W, "W", {"float8_e4m3fn", "uint8"});
    want_dtype(Y, "Y", {"bfloat16"});
    want_dtype(Xs, "X_scale", {"float32"});
    want_dtype(Ws, "W_scale", {"float32"});
    if (!bias.none) want_dtype(bias, "bias", {"float32"});
    for (const TView* t : {&gather, &hist, &offs, &data})
        if (!t->none) want_dtype(*t, t->name, {"int32"});
    if (group_k != 128 || group_n != 128) fail("group_k and group_n must be 128 (the block-scale granularity of this build)");
    if (X.rank() != 2 || X.dim(1) != K || Y.rank() != 2 || Y.dim(1) != N) fail("X must be [tokens, K] and Y [rows, N]");
    const int64_t tokens = X.dim(0), rows = Y.dim(0), E = hist.numel;
    if (W.numel != E * N * K) fail("W must hold E*N*K codes");
    if (stride_xk != 1 || stride_xm != K || stride_yn != 1 || stride_ym != N) fail("X and Y must be row-major and contiguous");
    if (stride_wk != 1 || stride_wn != K || stride_we != N * K)
        fail("W must be K-contiguous per output column: store the weights as [E, N, K] and pass the [E, K, N] view "
             "(stride_we = N*K, stride_wk = 1, stride_wn = K)");
    const int64_t kb = K / 128, nb = N / 128;
    if (Xs.numel != tokens * kb || stride_xsk != 1 || stride_xsm != kb) fail("X_scale must be contiguous [tokens, K/128]");
    if (Ws.numel != E * kb * nb || stride_wsn != 1 || stride_wsk != nb || stride_wse != kb * nb) fail("W_scale must be contiguous [E, K/128, N/128]");
    if (!bias.none && bias.numel != E * N) fail("bias must be [E, N]");
    if (offs.numel != E) fail("ExptOffs must have one entry per expert");
    if (data.numel < grid_m) fail("ExptData must have grid_m entries");
    if (!gather.none && gather.numel < rows) fail("GatherIndx must have one entry per output row");
    same_device({&X, &W, &Y, &Xs, &Ws, &bias, &gather, &hist, &offs, &data});
    Launch L(X.device);
    check(hkb_moe_gemm_fp8_blockscale(X.ptr, W.ptr, Y.ptr, (const float*)Xs.ptr, (const float*)Ws.ptr, bias.none ? nullptr : (const float*)bias.ptr,
                                      gather.none ? nullptr : (const int32_t*)gather.ptr, (const int32_t*)hist.ptr, (const int32_t*)offs.ptr,
                                      (const int32_t*)data.ptr, tokens, rows, E, N, K, grid_m, n_expts_act, L.stream));
}

// moe_op_mxfp4_tk.moe_mxfp4(...): kernels/moe-gemm/moe_op_mxfp4/kernel.cpp:262-349 -- same name, argument names and
// order.  Strides are checked, not used: A, C and A_mx_scale row-major; B and B_mx_scale K-contiguous per output
// column (the [E, K/2, N] / [E, K/32, N] views of [E, N, K/2] / [E, N, K/32] storage).
[[maybe_unused]] void moe_mxfp4(py::object A_, py::object B_, py::object C_, py::object Amx_, py::object Bmx_, py::object As_, py::object Bs_,
                                py::object tw_, py::object ids_, py::object eids_, int64_t N, int64_t K, int64_t num_valid_tokens,
                                int64_t top_k, bool mul_routed_weight, int64_t stride_am, int64_t stride_ak, int64_t stride_be,
                                int64_t stride_bk, int64_t stride_bn, int64_t stride_cm, int64_t stride_cn, int64_t stride_amxm,
                                int64_t stride_amxk, int64_t stride_bmxe, int64_t stride_bmxk, int64_t stride_bmxn, int64_t grid_m,
                                int64_t grid_n) {
    (void)grid_n;
    TView A = view(A_, "A"), B = view(B_, "B", false, false), C = view(C_, "C"), Amx = view(Amx_, "A_mx_scale"),
          Bmx = view(Bmx_, "B_mx_scale", false, false), As = view(As_, "A_scale", true), Bs = view(Bs_, "B_scale", true),
          tw = view(tw_, "topk_weights", true), ids = view(ids_, "sorted_token_ids"), eids = view(eids_, "expert_ids");
    want_dtype(A, "A", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(B, "B", {"uint8", "float4_e2m1fn_x2"});
    want_dtype(C, "C", {"bfloat16"});
    want_dtype(Amx, "A_mx_scale", {"uint8", "float8_e8m0fnu"});
    want_dtype(Bmx, "B_mx_scale", {"uint8", "float8_e8m0fnu"});
    for (const TView* t : {&As, &Bs, &tw})
        if (!t->none) want_dtype(*t, t->name, {"float32"});
    want_dtype(ids, "sorted_token_ids", {"int32"});
    want_dtype(eids, "expert_ids", {"int32"});
    if (K % 128 || A.rank() != 2 || A.dim(1) != K / 2 || C.rank() != 2 || C.dim(1) != N) fail("A must be [tokens, K/2] and C [rows, N], K a multiple of 128");
    const int64_t tokens = A.dim(0), num_padded = ids.numel;
    if (B.numel % (N * (K / 2))) fail("B must hold E*N*K/2 bytes");
    const int64_t E = B.numel / (N * (K / 2));
    if (eids.numel * 128 != num_padded || grid_m != eids.numel) fail("sorted_token_ids must hold 128 entries per entry of expert_ids (grid_m blocks)");
    if (C.dim(0) < num_valid_tokens) fail("C must have a row per valid (token, k) index");
    if (stride_ak != 1 || stride_am != K / 2 || stride_cn != 1 || stride_cm != N) fail("A and C must be row-major and contiguous");
    if (stride_bk != 1 || stride_bn != K / 2 || stride_be != N * (K / 2))
        fail("B must be K-contiguous per output column: store the weights as [E, N, K/2] and pass the [E, K/2, N] view "
             "(stride_be = N*K/2, stride_bk = 1, stride_bn = K/2)");
    if (Amx.numel != tokens * (K / 32) || stride_amxk != 1 || stride_amxm != K / 32) fail("A_mx_scale must be contiguous [tokens, K/32]");
    if (Bmx.numel != E * N * (K / 32) || stride_bmxk != 1 || stride_bmxn != K / 32 || stride_bmxe != N * (K / 32))
        fail("B_mx_scale must be K-contiguous per output column: [E, N, K/32] storage passed as the [E, K/32, N] view");
    if (!Bs.none && Bs.numel != E) fail("B_scale must have one entry per expert");
    if (mul_routed_weight && (tw.none || tw.numel < num_valid_tokens)) fail("topk_weights must have an entry per valid (token, k) index");
    same_device({&A, &B, &C, &Amx, &Bmx, &As, &Bs, &tw, &ids, &eids});
    Launch L(A.device);
    check(hkb_moe_gemm_mxfp4(A.ptr, B.ptr, C.ptr, Amx.ptr, Bmx.ptr, As.none ? nullptr : (const float*)As.ptr, Bs.none ? nullptr : (const float*)Bs.ptr,
                             tw.none ? nullptr : (const float*)tw.ptr, (const int32_t*)ids.ptr, (const int32_t*)eids.ptr, tokens, num_padded, E,
                             N, K, num_valid_tokens, top_k, mul_routed_weight ? 1 : 0, L.stream));
}

// quant_moe_tk: kernels/moe-misc/quant_moe/kernel.cpp:392-476 (same names, argument order and the
// redundant integer size arguments, which are checked against the tensors).
[[maybe_unused]] void downcast_to_static_fp8(py::object x_, py::object y_, py::object scale_, int64_t M, int64_t N) {
    TView x = view(x_, "x"), y = view(y_, "y"), sc = view(scale_, "scale");
    want_dtype(x, "x", {"bfloat16"});
    want_dtype(y, "y", {"float8_e4m3fn", "uint8"});
    want_dtype(sc, "scale", {"float32"});
    if (M < 0 || N < 0 || x.numel != M * N || y.numel != M * N) fail("x and y must have M*N elements");
    if (sc.numel < 1) fail("scale must hold one float");
    same_device({&x, &y, &sc});
    Launch L(x.device);
    check(hkb_moe_downcast_static_fp8(x.ptr, y.ptr, (const float*)sc.ptr, M, N, L.stream));
}
[[maybe_unused]] void downcast_to_mxfp(py::object t_, py::object s_, py::object src_, int64_t outer_dim, int64_t quant_dim, bool is_fp4) {
    TView t = view(t_, "mx_tensor"), sc = view(s_, "mx_scale"), src = view(src_, "src");
    want_dtype(src, "src", {"bfloat16"});
    want_dtype(t, "mx_tensor", {"uint8", "float8_e4m3fn", "float4_e2m1fn_x2"});
    want_dtype(sc, "mx_scale", {"uint8", "float8_e8m0fnu"});
    if (quant_dim <= 0 || quant_dim % 32) fail("quant_dim must be a positive multiple of 32");
    if (outer_dim < 0 || src.numel != outer_dim * quant_dim) fail("src must have outer_dim*quant_dim elements");
    if (t.numel != outer_dim * quant_dim / (is_fp4 ? 2 : 1)) fail("mx_tensor must have outer_dim*quant_dim (FP8) or half as many (FP4) bytes");
    if (sc.numel != outer_dim * (quant_dim / 32)) fail("mx_scale must have outer_dim*quant_dim/32 bytes");
    same_device({&t, &sc, &src});
    Launch L(src.device);
    check(hkb_moe_downcast_mxfp(t.ptr, sc.ptr, src.ptr, outer_dim, quant_dim, is_fp4 ? 1 : 0, L.stream));
}
[[maybe_unused]] void upcast_from_mxfp(py::object out_, py::object s_, py::object t_, int64_t outer_dim, int64_t quant_dim, bool is_fp4) {
    TView out = view(out_, "out"), sc = view(s_, "mx_scale"), t = view(t_, "mx_tensor");
    want_dtype(out, "out", {"bfloat16"});
    want_dtype(t, "mx_tensor", {"uint8", "float8_e4m3fn", "float4_e2m1fn_x2"});
    want_dtype(sc, "mx_scale", {"uint8", "float8_e8m0fnu"});
    if (quant_dim <= 0 || quant_dim % 32) fail("quant_dim must be a positive multiple of 32");
    if (outer_dim < 0 || out.numel != outer_dim * quant_dim) fail("out must have outer_dim*quant_dim elements");
    if (t.numel != outer_dim * quant_dim / (is_fp4 ? 2 : 1)) fail("mx_tensor must have outer_dim*quant_dim (FP8) or half as many (FP4) bytes");
    if (sc.numel != outer_dim * (quant_dim / 32)) fail("mx_scale must have outer_dim*quant_dim/32 bytes");
    same_device({&out, &sc, &t});
    Launch L(out.device);
    check(hkb_moe_upcast_mxfp(out.ptr, sc.ptr, t.ptr, outer_dim, quant_dim, is_fp4 ? 1 : 0, L.stream));
}

}  // namespace

#ifndef HKB_SHIM_NAME
#error "compile with -DHKB_SHIM_NAME=<module name>"
#endif

PYBIND11_MODULE(HKB_SHIM_NAME, m) {
    using namespace pybind11::literals;
#if defined(HKB_SHIM_QUANT)
    m.doc() = "per-token dynamic quantization (FP8 e4m3fn, or INT8 when output is int8), sm_100a";
    m.def("per_token_quant_fwd", &per_token_quant_fwd, "input"_a, "output"_a, "scales"_a);
#elif defined(HKB_SHIM_FUSED_FP8_QUANT)
    m.doc() = "1x128 block FP8 quantizer with optional fused RMSNorm; 128x128 weight quantizer, sm_100a";
    m.def("fused_rmsnorm_fp8_quant_fwd", &fused_rmsnorm_fp8_quant_fwd, "input"_a, "weight"_a, "output"_a, "scales"_a, "eps"_a = 1e-6f);
    m.def("weight_quant_128x128", &weight_quant_128x128, "weight"_a, "output"_a, "scales"_a);
#elif defined(HKB_SHIM_FUSED_MXFP4_QUANT)
    m.doc() = "MXFP4 (e2m1 + e8m0 per 32) quantizer with optional fused RMSNorm, sm_100a";
    m.def("fused_rmsnorm_mxfp4_quant_fwd", &fused_rmsnorm_mxfp4_quant_fwd, "input"_a, "weight"_a, "output"_a, "scales"_a,
          "eps"_a = 1e-6f, "mode"_a = py::none());
    m.def("fused_rmsnorm_mxfp4_quant_tc_fwd", &fused_rmsnorm_mxfp4_quant_tc_fwd, "input"_a, "weight"_a, "output"_a, "scales"_a,
          "sf_tc"_a, "eps"_a = 1e-6f, "mode"_a = py::none());
#elif defined(HKB_SHIM_GEMM_A8W8)
    m.doc() = "FP8 GEMM with per-row / per-channel scales (argument order A, B, a_scale, b_scale, C), sm_100a tcgen05";
    m.def("dispatch", &dispatch_a8w8, "A"_a, "B"_a, "a_scale"_a, "b_scale"_a, "C"_a);
#elif defined(HKB_SHIM_GEMM_A8W8_PER_TOKEN_SCALE)
    m.doc() = "FP8 GEMM with per-token / per-channel scales, sm_100a tcgen05";
    m.def("dispatch", &dispatch_per_token, "A"_a, "B"_a, "C"_a, "a_scale"_a, "b_scale"_a);
#elif defined(HKB_SHIM_GEMM_A8W8_BLOCKSCALE)
    m.doc() = "FP8 GEMM with 1x128 activation and 128x128 (or 128x1) weight block scales, sm_100a tcgen05";
    m.def("dispatch", &dispatch_blockscale, "A"_a, "B"_a, "C"_a, "a_scale"_a, "b_scale"_a);
    m.def("dispatch_scatter", &dispatch_blockscale_scatter, "A"_a, "B"_a, "dst_ptrs"_a, "ldc"_a, "a_scale"_a, "b_scale"_a);
    m.def("dispatch_timeline", &dispatch_blockscale_timeline, "A"_a, "B"_a, "C"_a, "a_scale"_a, "b_scale"_a, "trace"_a);
#elif defined(HKB_SHIM_GEMM_AFP4WFP4)
    m.doc() = "MXFP4 x MXFP4 GEMM (e2m1 codes, e8m0 scales per 32), sm_100a tcgen05 block-scaled MMA";
    m.def("dispatch", &dispatch_mxfp4, "A"_a, "B"_a, "C"_a, "a_scales"_a = py::none(), "b_scales"_a = py::none());
    m.def("sf_tc_bytes", &mxfp4_sf_tc_bytes, "batch"_a, "rows"_a, "K"_a);
    m.def("sf_to_tc", &mxfp4_sf_to_tc, "scales"_a, "sf_tc"_a, "K"_a);
    m.def("dispatch_tc", &dispatch_mxfp4_tc, "A"_a, "B"_a, "C"_a, "a_scales"_a, "b_scales"_a, "a_is_tc"_a, "b_is_tc"_a);
#elif defined(HKB_SHIM_BATCHED_GEMM_A8W8)
    m.doc() = "batched FP8 GEMM with per-token / per-channel scales and optional bias, sm_100a tcgen05";
    m.def("dispatch", &dispatch_batched_a8w8, "A"_a, "B"_a, "a_scale"_a, "b_scale"_a, "C"_a, "bias"_a = py::none());
#elif defined(HKB_SHIM_BATCHED_GEMM_A8W8_PTGQ)
    m.doc() = "batched FP8 GEMM with in-loop per-row, per-64-K-group activation quantization and a scalar weight scale, sm_100a tcgen05";
    m.def("dispatch", &dispatch_ptgq, "a"_a, "b"_a, "b_scale"_a, "c"_a, "bias"_a = py::none());
#elif defined(HKB_SHIM_BATCHED_GEMM_AFP4WFP4)
    m.doc() = "batched MXFP4 x MXFP4 GEMM, sm_100a tcgen05 block-scaled MMA";
    m.def("dispatch", &dispatch_mxfp4, "A"_a, "B"_a, "C"_a, "a_scales"_a = py::none(), "b_scales"_a = py::none());
#elif defined(HKB_SHIM_FUSED_GEMM_A8W8_BLOCKSCALE_MUL_ADD)
    m.doc() = "block-scale FP8 GEMM with fused multiply-add epilogue C = c_a * gemm + c_b, sm_100a tcgen05";
    m.def("dispatch", &dispatch_blockscale_mul_add, "a"_a, "b"_a, "c"_a, "a_scale"_a, "b_scale"_a, "c_a"_a, "c_b"_a);
#elif defined(HKB_SHIM_FUSED_GEMM_AFP4WFP4_MUL_ADD)
    m.doc() = "MXFP4 x MXFP4 GEMM with fused multiply-add epilogue C = c_a * gemm + c_b, sm_100a tcgen05";
    m.def("dispatch", &dispatch_mxfp4_mul_add, "a"_a, "b"_a, "c"_a, "a_scale"_a, "b_scale"_a, "c_a"_a, "c_b"_a);
#elif defined(HKB_SHIM_FUSED_GEMM_A8W8_BLOCKSCALE_SPLIT_CAT)
    m.doc() = "block-scale FP8 GEMM with the split-concatenate epilogue (c1, c2 written from the epilogue), sm_100a tcgen05";
    m.def("dispatch", &dispatch_blockscale_split_cat, "a"_a, "b"_a, "a_scale"_a, "b_scale"_a, "y"_a, "c1"_a, "c2"_a);
#elif defined(HKB_SHIM_FUSED_GEMM_AFP4WFP4_SPLIT_CAT)
    m.doc() = "MXFP4 x MXFP4 GEMM with the split-concatenate epilogue, sm_100a tcgen05";
    m.def("dispatch", &dispatch_mxfp4_split_cat, "a"_a, "b"_a, "a_scale"_a, "b_scale"_a, "y"_a, "c1"_a, "c2"_a);
#elif defined(HKB_SHIM_MOE_OP_GEMM_A8W8_BLOCKSCALE)
    m.doc() = "MoE grouped block-scale FP8 GEMM over expert-sorted rows, sm_100a tcgen05";
    m.def("moe_a8w8_blockscale", &moe_a8w8_blockscale, "X"_a, "W"_a, "Y"_a, "X_scale"_a, "W_scale"_a, "bias"_a, "GatherIndx"_a,
          "ExptHist"_a, "ExptOffs"_a, "ExptData"_a, "N"_a, "K"_a, "group_k"_a, "group_n"_a, "grid_m"_a, "grid_n"_a, "n_expts_act"_a,
          "stride_ym"_a, "stride_yn"_a, "stride_xm"_a, "stride_xk"_a, "stride_we"_a, "stride_wk"_a, "stride_wn"_a,
          "stride_xsm"_a, "stride_xsk"_a, "stride_wse"_a, "stride_wsk"_a, "stride_wsn"_a);
#elif defined(HKB_SHIM_MOE_OP_MXFP4)
    m.doc() = "MoE grouped MXFP4 x MXFP4 GEMM over a padded, expert-sorted row list, sm_100a tcgen05 block-scaled MMA";
    m.def("moe_mxfp4", &moe_mxfp4, "A"_a, "B"_a, "C"_a, "A_mx_scale"_a, "B_mx_scale"_a, "A_scale"_a, "B_scale"_a, "topk_weights"_a,
          "sorted_token_ids"_a, "expert_ids"_a, "N"_a, "K"_a, "num_valid_tokens"_a, "top_k"_a, "mul_routed_weight"_a, "stride_am"_a,
          "stride_ak"_a, "stride_be"_a, "stride_bk"_a, "stride_bn"_a, "stride_cm"_a, "stride_cn"_a, "stride_amxm"_a, "stride_amxk"_a,
          "stride_bmxe"_a, "stride_bmxk"_a, "stride_bmxn"_a, "grid_m"_a, "grid_n"_a);
#elif defined(HKB_SHIM_QUANT_MOE)
    m.doc() = "MoE casts: static FP8 down-cast, MX (e4m3 / e2m1 + exponent byte per 32) down- and up-cast, sm_100a";
    m.def("downcast_to_static_fp8", &downcast_to_static_fp8, "x"_a, "y"_a, "scale"_a, "M"_a, "N"_a);
    m.def("downcast_to_mxfp", &downcast_to_mxfp, "mx_tensor"_a, "mx_scale"_a, "src"_a, "outer_dim"_a, "quant_dim"_a, "is_fp4"_a);
    m.def("upcast_from_mxfp", &upcast_from_mxfp, "out"_a, "mx_scale"_a, "mx_tensor"_a, "outer_dim"_a, "quant_dim"_a, "is_fp4"_a);
#else
#error "unknown shim selector"
#endif
    m.def("hkb_version", []() { return hkb_version(); });
    m.def("hkb_last_kernel", []() { return std::string(hkb_last_kernel()); });
}
