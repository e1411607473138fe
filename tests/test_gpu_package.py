"""The qlinear4bit-compatible Python package on a GPU: module forwards against the CPU oracle
(bit-exact), buffer names of the reference's state_dict, the `qlinear4bit` import alias."""
import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    import qlinear4bit.nn as qnn                      # the alias a user of the reference imports
    import qlinear4bit.tools.tensor_utils as tu
    from oracle import oracle as o
    return torch, qnn, tu, o


def _lin(torch, K, N, seed, bias=True, std=0.02):
    g = torch.Generator().manual_seed(seed)
    lin = torch.nn.Linear(K, N, bias=bias)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(N, K, generator=g) * std)
        if bias:
            lin.bias.copy_(torch.randn(N, generator=g))
    return lin.half()


def test_alias_and_state_dict_names(env):
    torch, qnn, tu, o = env
    import duqlinear4bitcuda_b200.nn as impl
    assert qnn.Linear4bitSQ is impl.Linear4bitSQ
    assert sorted(qnn.Linear4bitSQ(64, 8, bias=True).state_dict()) == ["bias", "weight", "weight_scales"]
    assert sorted(qnn.Linear4bitDUSQ(64, 8).state_dict()) == ["weight", "weight_scales_1", "weight_scales_2"]
    assert sorted(qnn.Linear4bitASQ(64, 8, bias=True).state_dict()) == ["bias", "weight", "weight_scales", "weight_zeros"]
    assert sorted(qnn.LinearQuant4bitDUASQ(64, 8).state_dict()) == [
        "weight", "weight_scales_1", "weight_scales_2", "weight_zeros_1", "weight_zeros_2"]
    m = qnn.Linear4bitASQ(64, 8)
    assert m.weight.dtype == torch.uint8 and tuple(m.weight.shape) == (8, 32) and m.weight_scales.dtype == torch.float16
    assert tuple(m.weight_zeros.shape) == (8, 1)
    assert tu.get_dual_quant_col() == 10


@pytest.mark.parametrize("shape", [(3, 256), (2, 40, 256), (1, 300, 512)])
def test_sym_quantizer_and_linear(env, shape):
    torch, qnn, tu, o = env
    K, N = shape[-1], 136
    lin = _lin(torch, K, N, 1)
    w = lin.weight.data
    scales = (w.abs().amax(dim=1, keepdim=True).float() / 7).half()
    mod = qnn.Linear4bitSQ.from_float(lin, weight_scales=scales).cuda()
    quant = qnn.SymQuantizer(input_clip_ratio=0.9)
    x = torch.from_numpy(U.acts(int(np.prod(shape[:-1])), K, 3)).view(*shape).cuda()
    packed = quant(x)
    y = mod(packed)
    assert tuple(y.shape) == (*shape[:-1], N) and y.dtype == torch.float16
    # oracle pipeline
    x2 = x.view(-1, K).cpu().numpy()
    s = o.sym_scales(x2, 0.9)
    assert np.array_equal(packed.scales_x.reshape(-1).cpu().numpy().view(np.uint16), s.view(np.uint16))
    assert packed.scales_x.shape == ((shape[0], 1) if len(shape) == 2 else (shape[0], 1, shape[1]))   # the reference's unsqueeze(1)
    qa = packed.quantized_x.view(-1, K // 2).cpu().numpy()
    qw = mod.weight.cpu().numpy()
    _, want = o.linear_w4a4("sym", qa, qw, s, None, mod.weight_scales.cpu().numpy(), None, None, None,
                            mod.bias.cpu().numpy())
    assert U.f16_equal_nan(y.view(-1, N).cpu().numpy(), want)
    # the reference's three-call sequence through the functional wrappers gives the same tensor
    acc = tu.matmul(packed.quantized_x, mod.weight)
    y3 = tu.sym_dequant(acc, packed.scales_x, mod.weight_scales) + mod.bias
    assert torch.equal(y3.view(torch.int16), y.view(torch.int16))


def test_asym_modules(env, golden):
    torch, qnn, tu, o = env
    lin = _lin(torch, 128, 24, 5)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(golden["asq_w"])); lin.bias.copy_(torch.from_numpy(golden["asq_b"]))
    m = qnn.Linear4bitASQ.from_linear(lin, require_quantizer=True)
    assert np.array_equal(m.weight.numpy(), golden["asq_weight"])                   # reference's own from_linear output
    assert np.array_equal(m.weight_zeros.numpy().view(np.uint16), golden["asq_zeros"].view(np.uint16))
    d = qnn.LinearQuant4bitDUASQ.from_linear(lin, require_quantizer=True)
    assert np.array_equal(d.weight.numpy(), golden["duasq_weight"])
    for k in ("weight_scales_1", "weight_zeros_1", "weight_scales_2", "weight_zeros_2"):
        assert np.array_equal(getattr(d, k).numpy().view(np.uint16), golden["duasq_" + k].view(np.uint16))
    x = torch.from_numpy(U.acts(37, 128, 7, mean=0.1)).cuda()
    x2 = x.cpu().numpy()
    import duqlinear4bitcuda_b200.lib as L
    qa, s, z, _, _ = U.gpu_quantize(torch, L, "asym", x2)   # AsymQuantizer's codes, checked against the oracle
    for mod, mode in ((m.cuda(), "asym"), (d.cuda(), "asym_dual")):
        y = mod(x)
        sc1 = (mod.weight_scales if mode == "asym" else mod.weight_scales_1).cpu().numpy()
        zc1 = (mod.weight_zeros if mode == "asym" else mod.weight_zeros_1).cpu().numpy()
        sc2 = None if mode == "asym" else mod.weight_scales_2.cpu().numpy()
        zc2 = None if mode == "asym" else mod.weight_zeros_2.cpu().numpy()
        _, want = o.linear_w4a4(mode, qa, mod.weight.cpu().numpy(), s, z, sc1, zc1, sc2, zc2, mod.bias.cpu().numpy())
        assert U.f16_equal_nan(y.cpu().numpy(), want), mode


def test_dual_sym_module(env):
    torch, qnn, tu, o = env
    K, N = 192, 72
    lin = _lin(torch, K, N, 9, bias=False)
    w = lin.weight.data
    s1 = (w[:, :10].abs().amax(dim=1, keepdim=True).float() / 7).half()
    s2 = (w[:, 10:].abs().amax(dim=1, keepdim=True).float() / 7).half()
    mod = qnn.Linear4bitDUSQ.from_float(lin, s1, s2).cuda()
    x = torch.from_numpy(U.acts(20, K, 2)).cuda()
    packed = qnn.SymQuantizer()(x)
    y = mod(packed)
    qa = packed.quantized_x.cpu().numpy(); sa = packed.scales_x.reshape(-1).cpu().numpy()
    _, want = o.linear_w4a4("sym_dual", qa, mod.weight.cpu().numpy(), sa, None, s1.numpy(), None, s2.numpy(), None)
    assert U.f16_equal_nan(y.cpu().numpy(), want)


def test_quant_matmul_modules(env):
    torch, qnn, tu, o = env
    A = torch.from_numpy(U.acts(2 * 3 * 20, 128, 1, mean=0.1)).view(2, 3, 20, 128).cuda()
    B = torch.from_numpy(U.acts(2 * 3 * 24, 128, 2, mean=-0.1)).view(2, 3, 24, 128).cuda()
    C = qnn.AsymQuantMatMul()(A, B)
    assert tuple(C.shape) == (2, 3, 20, 24)
    a2 = A.view(6, 20, 128).cpu().numpy(); b2 = B.view(6, 24, 128).cpu().numpy()
    import duqlinear4bitcuda_b200.lib as L
    for i in range(6):
        qa, sa, za, _, _ = U.gpu_quantize(torch, L, "asym", a2[i]); qb, sb, zb, _, _ = U.gpu_quantize(torch, L, "asym", b2[i])
        want = o.asym_dequant(o.matmul_4bit(qa, qb), sa, za, sb, zb)
        assert U.f16_equal_nan(C.view(6, 20, 24)[i].cpu().numpy(), want), i
    S = qnn.SymQuantMatMul()(A[0, 0], B[0, 0])
    qa, sa, _, _, _ = U.gpu_quantize(torch, L, "sym", a2[0]); qb, sb, _, _, _ = U.gpu_quantize(torch, L, "sym", b2[0])
    want = o.sym_dequant(o.matmul_4bit(qa, qb), sa, sb)
    assert U.f16_equal_nan(S.cpu().numpy(), want)


def test_8bit_side_path(env):
    torch, qnn, tu, o = env
    lin = _lin(torch, 128, 40, 11).float()
    mod = qnn.LinearQuant8bitASQ.from_linear(lin).cuda()
    x = (torch.randn(33, 128, generator=torch.Generator().manual_seed(3)) * 2).cuda()
    y = mod(x)
    assert y.dtype == torch.float32 and tuple(y.shape) == (33, 40)
    q = mod.quantizer(x)
    acc = o.matmul_8bit(q.quantized_x.cpu().numpy(), mod.weight.cpu().numpy())
    want = o.asym_dequant_hprec(acc, q.scales_x.cpu().numpy(), q.zeros_x.cpu().numpy(), mod.weight_scales.cpu().numpy(),
                                mod.weight_zeros.cpu().numpy()) + mod.bias.cpu().numpy()
    assert np.array_equal(y.cpu().numpy(), want.astype(np.float32))


def test_operator_argument_checks(env):
    torch, qnn, tu, o = env
    import qlinear4bit._CUDA as ops
    x = torch.zeros((4, 64), dtype=torch.float16, device="cuda"); s = torch.ones(4, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.sym_quant(x.cpu(), s)                    # not a CUDA tensor
    with pytest.raises(RuntimeError):
        ops.sym_quant(x.t(), s)                      # not contiguous
    with pytest.raises(RuntimeError):
        ops.sym_quant(x, s[:3])                      # scale.size(0) != rows
    with pytest.raises(RuntimeError, match="Unsupported data type"):
        ops.sym_dequant(torch.zeros((4, 4), dtype=torch.int32, device="cuda"), s, s, 16)
    with pytest.raises(AssertionError):
        tu.matmul(torch.zeros((4, 24), dtype=torch.uint8, device="cuda"), torch.zeros((4, 24), dtype=torch.uint8, device="cuda"))
    q = ops.asym_dual_quant(x, s, s, s, s)           # returns its tensor (the reference's binding does not)
    assert q.dtype == torch.uint8 and tuple(q.shape) == (4, 32)
    # dtypes are checked, not reinterpreted: fp32 scales, an fp32 bias or bf16 activations would otherwise be read
    # as fp16 bit patterns and give silently wrong numbers
    w = torch.zeros((8, 32), dtype=torch.uint8, device="cuda"); sc = torch.ones(8, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="dtype"):
        ops.sym_quant(x, s.float())
    with pytest.raises(RuntimeError, match="dtype"):
        ops.sym_quant(x.to(torch.bfloat16), s)
    with pytest.raises(RuntimeError, match="dtype"):
        ops.linear_w4a4("sym", q, w, s, None, sc.float())
    with pytest.raises(RuntimeError, match="dtype"):
        ops.linear_w4a4("sym", q, w, s, None, sc, bias=torch.zeros(8, device="cuda"))
    with pytest.raises(RuntimeError, match="dtype"):
        ops.linear_w4a4("sym", q.to(torch.int8), w, s, None, sc)
    with pytest.raises(RuntimeError):
        ops.linear_w4a4_from_fp16("sym", x.float(), w, sc)
    with pytest.raises(RuntimeError, match="dtype"):
        ops.linear_w4a4_from_fp16("sym", x, w, sc.float())
    with pytest.raises(RuntimeError, match="dtype"):
        ops.quantize_sym_fused(x.float())
    with pytest.raises(RuntimeError, match="dtype"):
        ops.linear_w4a4_batched("asym", q.view(1, 4, 32), w.view(1, 8, 32), s.view(1, 4), s.view(1, 4), sc.view(1, 8).float(), sc.view(1, 8))
    with pytest.raises(RuntimeError, match="unknown mode"):
        ops.linear_w4a4("symm", q, w, s, None, sc)


def test_module_weight_prelayout_cache(env):
    """A module that owns its quantizer runs forwards of >= 256 tokens on a lazily built int8 copy of its packed
    weights: same output bits as with the cache disabled, the copy is rebuilt when the weights change, and the
    state_dict is unaffected."""
    torch, qnn, tu, o = env
    lin = _lin(torch, 256, 72, 31)
    m = qnn.Linear4bitASQ.from_linear(lin, require_quantizer=True).cuda()
    x = torch.from_numpy(U.acts(300, 256, 5, mean=0.1)).cuda()
    y_cached = m(x)
    assert "_prelaid" in m.__dict__ and m.__dict__["_prelaid"][1].dtype == torch.int8 and tuple(m.__dict__["_prelaid"][1].shape) == (72, 256)
    m.weight_prelayout = False
    y_plain = m(x)
    assert torch.equal(y_cached.view(torch.int16), y_plain.view(torch.int16))
    m.weight_prelayout = True
    assert m(x[:8]).shape == (8, 72) and torch.equal(m(x[:8]).view(torch.int16), y_plain[:8].view(torch.int16))   # few tokens: packed weights
    with torch.no_grad():
        m.weight.copy_(torch.randint(0, 256, m.weight.shape, dtype=torch.uint8))   # in-place change -> new version -> rebuilt copy
    y_new = m(x)
    m.weight_prelayout = False
    assert torch.equal(y_new.view(torch.int16), m(x).view(torch.int16)) and not torch.equal(y_new, y_cached)
    assert sorted(m.state_dict()) == ["bias", "weight", "weight_scales", "weight_zeros"]


def test_module_with_fp32_scale_buffers_matches_fp16(env):
    """Linear4bitSQ registers weight_scales with torch's default dtype (fp32), as the reference does; a module
    built directly and filled by load_state_dict keeps them in fp32. The forward converts them once and gives
    the same output as the from_float module (fp16 scales)."""
    torch, qnn, tu, o = env
    lin = _lin(torch, 256, 72, 21)
    scales = (lin.weight.data.abs().amax(dim=1, keepdim=True).float() / 7).half()
    a = qnn.Linear4bitSQ.from_float(lin, weight_scales=scales).cuda()
    b = qnn.Linear4bitSQ(256, 72, bias=True)
    assert b.weight_scales.dtype == torch.float32
    b.load_state_dict(a.state_dict())
    b = b.cuda()
    assert b.weight_scales.dtype == torch.float32
    packed = qnn.SymQuantizer()(torch.from_numpy(U.acts(20, 256, 5)).cuda())
    ya, yb = a(packed), b(packed)
    assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))
    assert torch.equal(b(packed).view(torch.int16), ya.view(torch.int16))   # second call: cached fp16 copy


@pytest.mark.parametrize("rows,inter", [(5, 64), (33, 11008), (300, 1024)])
def test_silu_mul_quantize_fused_equals_torch_composition(env, rows, inter):
    """SiLU-gated MLP glue: the fused kernel's scales and codes equal quantizing the fp16 tensor
    F.silu(gate) * up that torch produces (the composition a user of the reference writes)."""
    torch, qnn, tu, o = env
    import qlinear4bit._CUDA as ops
    g = torch.Generator(device="cuda").manual_seed(rows)
    gate_up = (torch.randn((rows, 2 * inter), device="cuda", generator=g) * 3).half()
    h = (torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]).contiguous()
    q_ref, s_ref = ops.quantize_sym_fused(h, 0.95)
    q, s = ops.silu_mul_quantize_fused(gate_up, "sym", 0.95)
    assert torch.equal(s.view(torch.int16), s_ref.view(torch.int16))
    assert torch.equal(q, q_ref)
    qa_ref, sa_ref, za_ref = ops.quantize_asym_fused(h)
    qa, sa, za = ops.silu_mul_quantize_fused(gate_up, "asym")
    assert torch.equal(sa.view(torch.int16), sa_ref.view(torch.int16)) and torch.equal(za.view(torch.int16), za_ref.view(torch.int16))
    assert torch.equal(qa, qa_ref)
    # and against the CPU oracle on the stored h
    hn = h.cpu().numpy()
    assert np.array_equal(s.cpu().numpy().view(np.uint16), o.sym_scales(hn, 0.95).view(np.uint16))
    if inter % 64 == 0:   # tensor-core-ready int8 output feeds the GEMM directly
        q8, s8 = ops.silu_mul_quantize_fused(gate_up, "sym", 0.95, tensor_core_ready=True)
        codes = o.unpack_s4(q.cpu().numpy()).astype(np.int16)
        pos = np.arange(inter); blk, r = pos // 128, pos % 128
        src = blk * 128 + 32 * (r // 32) + 2 * (r % 16) + ((r % 32) // 16)
        assert np.array_equal(q8.cpu().numpy().astype(np.int16), 16 * codes[:, src])


def test_owned_quantizer_modules_fp16_path_equals_two_step_path(env):
    """Linear4bitASQ / LinearQuant4bitDUASQ given fp16 input run quantize+GEMM+dequant in one call;
    the result equals quantizer module -> linear on the packed tensor, bit for bit."""
    torch, qnn, tu, o = env
    lin = _lin(torch, 512, 264, 21)
    x = torch.from_numpy(U.acts(2 * 150, 512, 22, mean=0.1)).view(2, 150, 512).cuda()
    for cls in (qnn.Linear4bitASQ, qnn.LinearQuant4bitDUASQ):
        mod = cls.from_linear(lin, require_quantizer=True).cuda()
        y = mod(x)
        packed = mod.quantizer(x)
        y2 = mod._fused(packed)
        assert tuple(y.shape) == (2, 150, 264)
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16)), cls.__name__


@pytest.mark.parametrize("mode,M", [("sym", 5), ("sym", 300), ("asym", 40)])
def test_row_parallel_layer_single_rank_equals_fused_layer(mode, M):
    """RowParallelLinear4bit without a process group (one K-slice = the whole K): its piecewise path
    (torch statistics, quantize with a given scale, int32 GEMM, dequant) must equal the one-call
    fused layer bit for bit -- the same identity the multi-rank form relies on."""
    import torch
    from duqlinear4bitcuda_b200.parallel import ColumnParallelLinear4bit, RowParallelLinear4bit
    N, K = 520, 1024
    x = torch.from_numpy(U.acts(M, K, 31, mean=0.1 if mode == "asym" else 0.0)).cuda()
    t = lambda a: torch.from_numpy(a).cuda()
    qw = t(U.rand_codes(N, K, 32)); sc = t(U.rand_scales(N, 33)); zc = t(U.rand_zeros(N, 34))
    bias = t(np.random.default_rng(35).standard_normal(N).astype(np.float16))
    row = RowParallelLinear4bit.from_full(mode, qw, sc, zc if mode == "asym" else None, bias)
    col = ColumnParallelLinear4bit(mode, N, qw, sc, zc if mode == "asym" else None, None, None, bias, unsharded=True)
    y_row, y_col = row(x), col(x)
    torch.cuda.synchronize()
    assert tuple(y_row.shape) == (M, N)
    assert torch.equal(y_row.view(torch.int16), y_col.view(torch.int16))
    with pytest.raises(ValueError):
        RowParallelLinear4bit.from_full("sym_dual", qw, sc)


@pytest.mark.parametrize("mode,M,inter,K,int8_acts", [("sym", 300, 1408, 512, True), ("asym", 64, 200, 448, False),
                                                      ("sym", 2048, 2816, 1024, True), ("asym", 520, 1408, 512, True)])
def test_gate_up_silu_epilogue_equals_unfused_composition(mode, M, inter, K, int8_acts):
    """One-launch SiLU-gated gate/up projection == linear_w4a4 on the fused [2*I, K] weight followed by
    torch's F.silu(gate) * up, bit for bit (ragged M, I not a multiple of the 128-channel tile, bias,
    both activation formats, asymmetric epilogue)."""
    import torch
    import qlinear4bit._CUDA as ops
    import duqlinear4bitcuda_b200.lib as L
    t = lambda a: torch.from_numpy(a).cuda()
    x = t(U.acts(M, K, 51, mean=0.1 if mode == "asym" else 0.0))
    qw = t(U.rand_codes(2 * inter, K, 52))
    sc = t(U.rand_scales(2 * inter, 53, 0.002, 0.02)); zc = t(U.rand_zeros(2 * inter, 54))
    bias = t((np.random.default_rng(55).standard_normal(2 * inter) * 0.5).astype(np.float16))
    if mode == "sym":
        qa, sa = ops.quantize_sym_fused(x, 1.0); za = None
    else:
        qa, sa, za = ops.quantize_asym_fused(x)
    y = ops.linear_w4a4(mode, qa, qw, sa, za, sc, zc if mode == "asym" else None, None, None, bias)
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    A = qa
    if int8_acts:   # tensor-core-ready int8 activations from the fused quantizer
        A = torch.empty((M, K), dtype=torch.int8, device="cuda")
        s2 = torch.empty(M, dtype=torch.float16, device="cuda"); z2 = torch.empty(M, dtype=torch.float16, device="cuda")
        L.call("duq4_quantize_fused_i8", L.MODES[mode], L.ptr(x), M, K, 1.0, L.ptr(A), L.ptr(s2), L.ptr(z2) if mode == "asym" else None,
               None, None, L.current_stream())
        assert torch.equal(s2.view(torch.int16), sa.reshape(-1).view(torch.int16))
    h = ops.linear_w4a4_gate_up_silu(mode, A, qw, sa.reshape(-1), None if za is None else za.reshape(-1), sc,
                                     zc if mode == "asym" else None, bias)
    torch.cuda.synchronize()
    assert tuple(h.shape) == (M, inter)
    assert torch.equal(h.view(torch.int16), want.contiguous().view(torch.int16))
    with pytest.raises(RuntimeError):
        ops.linear_w4a4_gate_up_silu("sym_dual", A, qw, sa.reshape(-1), None, sc)
    if int8_acts and K % 128 == 0:   # the same on the pre-laid-out int8 copy of the fused gate/up weight
        import ctypes
        w8 = ops.weight_prelayout_i8(qw)
        h8 = torch.full((M, inter), float("nan"), dtype=torch.float16, device="cuda")
        epi = L.make_epilogue(mode, sa.reshape(-1), None if za is None else za.reshape(-1), sc, zc if mode == "asym" else None, None, None, bias)
        L.call("duq4_linear_w4a4_gate_up_silu_prelaid", L.ptr(A), L.ptr(w8), M, inter, K, ctypes.byref(epi), L.ptr(h8), L.current_stream())
        torch.cuda.synchronize()
        assert torch.equal(h8.view(torch.int16), want.contiguous().view(torch.int16))
        hb = ops.linear_w4a4_gate_up_silu(mode, A, qw, sa.reshape(-1), None if za is None else za.reshape(-1), sc,
                                          zc if mode == "asym" else None, bias, W_prelaid=w8)
        assert torch.equal(hb.view(torch.int16), want.contiguous().view(torch.int16))
