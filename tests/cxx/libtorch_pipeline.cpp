// libtorch parity program for include/linear.h and include/quant_tensor.h.
// Builds Quantizer4bit -> Linear4bit / Linear4bitDUQ (as the reference's test/pipeline.cu does) and
// checks the module outputs bit for bit against the REFERENCE'S OWN CUDA launchers, loaded from the
// checker library that oracle/Makefile (target `ref`) compiles from the reference's sources:
//   torch ops for the per-token scale (src/module/quant_tensor.cu:151-161)
//   -> sym_quant_host (src/kernels/quant.cu:48-61) -> matmul_host_4bit (src/kernels/gemm.cu:8-43)
//   -> sym_dequant_host / sym_dual_dequant_host (src/kernels/quant.cu:83-97, quant2.cu:85-98) -> + bias
// i.e. the chain of src/module/linear.cu:108-153 and :200-246. The library's tensor-level functions
// (sym_quant, sym_dequant, sym_dual_dequant of quant_tensor.h) are checked against the same launchers.
// usage: libtorch_pipeline <path to libduq_ref.so>; exit 0 = all equal, 3 = checker library missing.
#include <dlfcn.h>

#include <cstdio>

#include "gemm.h"
#include "linear.h"

typedef int (*RefQuant)(const void *, const void *, uint32_t, uint32_t, uint32_t, void *);
typedef int (*RefMatmul)(const void *, const void *, uint32_t, uint32_t, uint32_t, int32_t *);
typedef int (*RefDequant)(const int32_t *, const void *, const void *, uint32_t, uint32_t, void *);
typedef int (*RefDualDequant)(const int32_t *, const void *, const void *, const void *, uint32_t, uint32_t, void *);

static bool same_bits(const torch::Tensor &a, const torch::Tensor &b) {
    return a.sizes() == b.sizes() && torch::equal(a.contiguous().view(torch::kInt16), b.contiguous().view(torch::kInt16));
}

int main(int argc, char **argv) {
    if (!torch::cuda::is_available()) {
        std::printf("no CUDA device\n");
        return 2;
    }
    void *h = argc > 1 ? dlopen(argv[1], RTLD_NOW | RTLD_LOCAL) : nullptr;
    if (!h) {
        std::printf("reference checker library not available: %s\n", argc > 1 ? dlerror() : "no path given");
        return 3;
    }
    auto ref_sym_quant = (RefQuant)dlsym(h, "ref_sym_quant");
    auto ref_matmul = (RefMatmul)dlsym(h, "ref_matmul_4bit");
    auto ref_sym_dequant = (RefDequant)dlsym(h, "ref_sym_dequant");
    auto ref_sym_dual_dequant = (RefDualDequant)dlsym(h, "ref_sym_dual_dequant");
    if (!ref_sym_quant || !ref_matmul || !ref_sym_dequant || !ref_sym_dual_dequant) {
        std::printf("reference checker library lacks a launcher\n");
        return 3;
    }
    torch::manual_seed(0);
    const int64_t K = 512, N = 264;
    int failures = 0;
    auto fail = [&](const char *what, int64_t batch) { std::printf("%s (batch %ld)\n", what, (long)batch); ++failures; };
    const auto f16 = torch::dtype(torch::kFloat16).device(torch::kCUDA);
    for (int64_t batch : {4, 40}) {
        torch::nn::Linear lin(torch::nn::LinearOptions(K, N).bias(true));
        lin->to(torch::kCUDA, torch::kFloat16);
        auto w = lin->weight.data();
        auto x = torch::randn({batch, 3, K}, f16);
        auto x2 = x.view({-1, K}).contiguous();
        const uint32_t M = x2.size(0);

        // ---- the library's modules: single-scale symmetric and dual-uniform symmetric
        auto ws = (w.abs().amax(1, true).to(torch::kFloat32) / 7.0).to(torch::kFloat16);
        Quantizer4bit quant(0.9f);
        auto lin4 = Linear4bit::from_float(lin, ws);
        auto packed = quant.forward(x);
        auto y = lin4.forward(packed);
        using namespace torch::indexing;
        auto s1 = (w.index({Slice(), Slice(None, 10)}).abs().amax(1, true).to(torch::kFloat32) / 7.0).to(torch::kFloat16);
        auto s2 = (w.index({Slice(), Slice(10, None)}).abs().amax(1, true).to(torch::kFloat32) / 7.0).to(torch::kFloat16);
        auto duq = Linear4bitDUQ::from_float(lin, s1, s2);
        auto yd = duq.forward(packed);
        // ... and its tensor-level functions on the same operands
        auto scales = ((std::get<0>(torch::max(torch::abs(x), -1)).unsqueeze(1) / 7.0).to(torch::kFloat16) * 0.9).contiguous();
        auto q_lib = sym_quant(x2, scales.view(-1));
        torch::cuda::synchronize();

        // ---- the reference's launchers (legacy default stream; each wrapper synchronises the device)
        auto q_ref = torch::zeros({M, K / 2}, torch::dtype(torch::kUInt8).device(torch::kCUDA));
        auto acc = torch::zeros({M, N}, torch::dtype(torch::kInt32).device(torch::kCUDA));
        auto out = torch::zeros({M, N}, f16);
        auto outd = torch::zeros({M, N}, f16);
        auto sflat = scales.view(-1).contiguous();
        torch::cuda::synchronize();
        int rc = ref_sym_quant(x2.data_ptr(), sflat.data_ptr(), M, K, K / 2, q_ref.data_ptr());
        rc |= ref_matmul(q_ref.data_ptr(), lin4.weight.data_ptr(), M, N, K, acc.data_ptr<int32_t>());
        rc |= ref_sym_dequant(acc.data_ptr<int32_t>(), sflat.data_ptr(), lin4.weight_scale.data_ptr(), M, N, out.data_ptr());
        if (rc) fail("a reference launcher reported an error", batch);
        auto ref = out + lin4.bias;   // src/module/linear.cu:147-150
        auto y3 = sym_dequant(acc, sflat, lin4.weight_scale.view(-1), 32) + lin4.bias;
        auto acc_d = torch::zeros_like(acc);
        rc = ref_matmul(q_ref.data_ptr(), duq.weight.data_ptr(), M, N, K, acc_d.data_ptr<int32_t>());
        rc |= ref_sym_dual_dequant(acc_d.data_ptr<int32_t>(), sflat.data_ptr(), duq.weight_scale_1.data_ptr(),
                                   duq.weight_scale_2.data_ptr(), M, N, outd.data_ptr());
        if (rc) fail("a reference launcher reported an error (dual)", batch);
        auto refd = outd + duq.bias;
        auto yd3 = sym_dual_dequant(acc_d, sflat, duq.weight_scale_1.view(-1), duq.weight_scale_2.view(-1), 32) + duq.bias;

        if (!same_bits(packed.scale, scales)) fail("Quantizer4bit scales differ from the reference's torch chain", batch);
        if (!torch::equal(packed.quantized_x.view({-1, K / 2}), q_ref)) fail("Quantizer4bit codes differ from sym_quant_host", batch);
        if (!torch::equal(q_lib, q_ref)) fail("sym_quant differs from sym_quant_host", batch);
        if (!same_bits(y.view({-1, N}), ref)) fail("Linear4bit output differs from the reference's launch chain", batch);
        if (!same_bits(y3, ref)) fail("sym_dequant differs from sym_dequant_host", batch);
        if (!same_bits(yd.view({-1, N}), refd)) fail("Linear4bitDUQ output differs from the reference's launch chain", batch);
        if (!same_bits(yd3, refd)) fail("sym_dual_dequant differs from sym_dual_dequant_host", batch);
        if (y.sizes() != torch::IntArrayRef({batch, 3, N})) fail("output shape", batch);
    }
    std::printf(failures ? "FAILED %d\n" : "libtorch pipeline ok\n", failures);
    return failures ? 1 : 0;
}
