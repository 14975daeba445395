"""CPU-side checks: the C ABI library loads and exports every declared symbol, the package
surface matches the reference's, the host-side contract raises the reference's errors."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from rosa_soft_b200 import cabi
    header = open(os.path.join(ROOT, "include", "rosa_soft_b200.h")).read()
    declared = set(re.findall(r"ROSA_B200_API[^;(]*?\b(rosa_b200_\w+)\s*\(", header))
    assert declared == set(cabi.EXPORTED_SYMBOLS)
    lib = ctypes.CDLL(cabi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert cabi.load().rosa_b200_abi_version() == 1


def test_workspace_sizes_are_pure_functions_of_shapes():
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    a = lib.rosa_b200_surrogate_vjp_workspace_bytes(2 * 1024, 64, 8, 16, 8, 2, 1024, 128, 7)
    b = lib.rosa_b200_surrogate_vjp_workspace_bytes(2 * 1024, 64, 8, 16, 8, 2, 1024, 128, 7)
    assert a == b and a > 0
    # masked-off gradients need no partial buffers
    assert lib.rosa_b200_surrogate_vjp_workspace_bytes(2 * 1024, 64, 8, 16, 8, 2, 1024, 128, 4) < a
    # the packed bound grows with the token count, never reads offsets
    small = lib.rosa_b200_surrogate_vjp_workspace_bytes(4096, 4, 8, 2, 8, 16, 0, 64, 7)
    large = lib.rosa_b200_surrogate_vjp_workspace_bytes(8192, 4, 8, 2, 8, 16, 0, 64, 7)
    assert 0 < small < large


def test_status_word_decoding():
    """The plan's code wins; a set tensor-core word alone reads as the timeout status."""
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    assert lib.rosa_b200_decode_status(0, 0) == 0
    for code in (1, 2, 3, 4):
        assert lib.rosa_b200_decode_status(code, 0) == code
        assert lib.rosa_b200_decode_status(code, 1) == code
    assert lib.rosa_b200_decode_status(0, 1) == 5      # ROSA_B200_STATUS_MMA_TIMEOUT
    header = open(os.path.join(ROOT, "include", "rosa_soft_b200.h")).read()
    assert re.search(r"ROSA_B200_STATUS_MMA_TIMEOUT\s*=\s*5", header)


def test_argument_errors_without_a_gpu():
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    rc = lib.rosa_b200_hard_forward(None, None, None, 0, 8, 2, 40, 1, 3, None, 1, 8, 4, None, None,
                                    None, None, None, 0, None)
    assert rc != 0 and "bit dimension must be in [1, 32]" in cabi.last_error()
    rc = lib.rosa_b200_hard_forward(None, None, None, 0, 8, 3, 4, 2, 3, None, 1, 8, 4, None, None,
                                    None, None, None, 0, None)
    assert rc != 0 and "divisible by value heads" in cabi.last_error()


def test_package_surface_and_schemas():
    import rosa_soft_b200 as pkg
    caps = pkg.BUILD_CAPABILITIES
    assert (caps.variant, caps.compiled_extension, caps.rosa_soft_cuda) == ("cuda", True, True)
    with pytest.raises(Exception):
        caps.variant = "x"
    for name in ("rosa_soft", "rosa_soft_varlen", "BUILD_CAPABILITIES", "__version__"):
        assert name in pkg.__all__
    want = {
        "hard_forward": "rosa_soft::hard_forward(Tensor query, Tensor key, Tensor value, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)",
        "hard_forward_varlen": "rosa_soft::hard_forward_varlen(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)",
        "surrogate_vjp_masked": "rosa_soft::surrogate_vjp_masked(Tensor query, Tensor key, Tensor value, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)",
        "surrogate_vjp_varlen_masked": "rosa_soft::surrogate_vjp_varlen_masked(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)",
    }
    for op, schema in want.items():
        assert str(getattr(torch.ops.rosa_soft, op).default._schema) == schema
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"rosa_soft::{op}", "CUDA")
        assert not torch._C._dispatch_has_kernel_for_dispatch_key(f"rosa_soft::{op}", "CPU")


def test_no_cpu_fallback():
    import rosa_soft_b200 as pkg
    q = torch.randn(1, 4, 1, 2)
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        pkg.rosa_soft(q, q, q)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.rosa_soft.hard_forward(q, q, q, 2)


def test_validation_matrix():
    from rosa_soft_b200 import soft_contract as sc
    q = torch.randn(2, 6, 4, 3)
    v = torch.randn(2, 6, 2, 5)
    assert sc.validate_rosa_soft_inputs(q, q, v, 32, 1.0, 0.0, 3.0) == 6
    assert sc.validate_rosa_soft_inputs(q, q, v, 4, 1.0, 0.0, 3.0) == 4
    cases = [
        (dict(max_suffix_length=True), TypeError, "must be an integer"),
        (dict(max_suffix_length=1.5), TypeError, "must be an integer"),
        (dict(max_suffix_length=0), ValueError, ">= 1"),
        (dict(scale=float("inf")), ValueError, "scale must be finite"),
        (dict(scale=True), ValueError, "scale must be finite"),
        (dict(dropout_p=1.0), ValueError, "dropout_p must be finite"),
        (dict(dropout_p=-0.1), ValueError, "dropout_p must be finite"),
        (dict(mismatch_scale=0.0), ValueError, "mismatch_scale must be finite"),
    ]
    base = dict(max_suffix_length=8, scale=1.0, dropout_p=0.0, mismatch_scale=3.0)
    for override, exc, text in cases:
        kw = {**base, **override}
        with pytest.raises(exc, match=text):
            sc.validate_rosa_soft_inputs(q, q, v, kw["max_suffix_length"], kw["scale"],
                                         kw["dropout_p"], kw["mismatch_scale"])
    with pytest.raises(ValueError, match="divisible by value heads"):
        sc.validate_rosa_soft_inputs(q, q, torch.randn(2, 6, 3, 5), 8, 1.0, 0.0, 3.0)
    with pytest.raises(ValueError, match=r"in \[1, 32\]"):
        sc.validate_rosa_soft_inputs(torch.randn(1, 2, 1, 33), torch.randn(1, 2, 1, 33),
                                     torch.randn(1, 2, 1, 1), 8, 1.0, 0.0, 3.0)
    with pytest.raises(ValueError, match="same dtype"):
        sc.validate_rosa_soft_inputs(q, q.double(), v, 8, 1.0, 0.0, 3.0)
    qv, vv = torch.randn(10, 2, 3), torch.randn(10, 1, 2)
    good = torch.tensor([0, 4, 10], dtype=torch.int32)
    assert sc.validate_rosa_soft_varlen_inputs(qv, qv, vv, good, 64, 1.0, 0.0, 3.0) == 10
    for bad, text in ((torch.tensor([1, 4, 10], dtype=torch.int32), "start at zero"),
                      (torch.tensor([0, 4, 9], dtype=torch.int32), "end at the packed token count"),
                      (torch.tensor([0, 6, 4, 10], dtype=torch.int32), "nondecreasing"),
                      (torch.tensor([0, 10], dtype=torch.int64), "dtype int32")):
        with pytest.raises(ValueError, match=text):
            sc.validate_rosa_soft_varlen_inputs(qv, qv, vv, bad, 8, 1.0, 0.0, 3.0)
    with pytest.raises(ValueError, match="max_suffix_length \\* scale must fit"):
        sc.validate_fp32_surrogate_scalars(1 << 20, 3e38, 0.0, 3.0)
    seed = sc.make_dropout_seed(q, 0.0, True)
    assert seed.numel() == 0 and seed.dtype == torch.int64
    assert sc.make_dropout_seed(q, 0.5, False).numel() == 0
    assert sc.make_dropout_seed(q, 0.5, True).shape == ()


def test_runtime_constructor_and_input_contract_without_a_gpu():
    """Mirrors the argument errors of the reference runtime (rosa_soft/runtime.py:320-352,
    165-239); none of them needs a device."""
    from rosa_soft_b200 import RosaRuntime
    from rosa_soft_b200.runtime import pack_sign_bits, unpack_sign_bits
    with pytest.raises(ValueError, match=r"qk_bits must be in \[1, 8\]"):
        RosaRuntime(4, qk_bits=9)
    with pytest.raises(ValueError, match=r"payload_bits must be in \[1, 8\]"):
        RosaRuntime(4, payload_bits=0)
    with pytest.raises(TypeError, match="num_heads must be an integer"):
        RosaRuntime(True)
    with pytest.raises(ValueError, match="divisible"):
        RosaRuntime(4, 3)
    rt = RosaRuntime(4, 2, 3, 5, 16)
    assert (rt.num_heads, rt.num_payload_heads, rt.qk_bits, rt.payload_bits,
            rt.max_suffix_length, rt.state) == (4, 2, 3, 5, 16, "OPEN")
    u8 = lambda *shape: torch.zeros(shape, dtype=torch.uint8)
    with pytest.raises(TypeError, match="dtype torch.uint8"):
        rt.update_packed(u8(1, 2, 4).int(), u8(1, 2, 4), u8(1, 2, 2))
    with pytest.raises(ValueError, match="shapes differ"):
        rt.update_packed(u8(1, 2, 4), u8(1, 3, 4), u8(1, 2, 2))
    with pytest.raises(ValueError, match=r"\[B, T, H\]"):
        rt.update_packed(u8(2, 4), u8(2, 4), u8(2, 2))
    with pytest.raises(ValueError, match="CUDA tensors"):
        rt.update_packed(u8(1, 2, 4), u8(1, 2, 4), u8(1, 2, 2))
    with pytest.raises(ValueError, match="last dimension must equal qk_bits"):
        rt.update(torch.zeros(1, 2, 4, 2), torch.zeros(1, 2, 4, 2), torch.zeros(1, 2, 2, 5))
    x = torch.tensor([[0.5, -1.0, 0.0, 2.0, float("nan")]])
    packed = pack_sign_bits(x)
    assert packed.tolist() == [0b01001]                      # zero and NaN are not positive
    assert unpack_sign_bits(packed, 5, torch.float32).tolist() == [[1.0, -1.0, -1.0, 1.0, -1.0]]
    rt.close()
    rt.close()
    with pytest.raises(RuntimeError, match="closed"):
        rt.reset()


def test_installer_honours_the_reference_build_switches():
    """ROSA_BUILD_EXTENSION / USE_CUDA as in the reference's setup.py:50-96; the variants this
    package does not have are refused instead of installed half."""
    import types
    source = open(os.path.join(ROOT, "setup.py")).read()
    # run the script with `setup(...)` made a no-op: only its helpers are wanted here
    source = source.replace("from setuptools import setup\n", "setup = lambda **kw: None\n")
    module = types.ModuleType("_rosa_setup")
    module.__file__ = os.path.join(ROOT, "setup.py")
    exec(compile(source, module.__file__, "exec"), module.__dict__)
    assert module.resolve_variant({}) == "cuda"
    assert module.resolve_variant({"USE_CUDA": "1", "ROSA_BUILD_EXTENSION": "1"}) == "cuda"
    for env in ({"ROSA_BUILD_EXTENSION": "0"}, {"USE_CUDA": "0"}):
        with pytest.raises(RuntimeError, match="only exists as the CUDA variant"):
            module.resolve_variant(env)
    with pytest.raises(RuntimeError, match="USE_CUDA must be"):
        module.resolve_variant({"USE_CUDA": "maybe"})
    assert module._version() == "0.1.0"


def test_symbol_health_and_route_summary_on_cpu():
    """The statistics helpers of the inspection module are plain tensor reductions: checked on
    CPU against their definitions (reference rosa_soft/diagnostics.py:186-207, 264-274)."""
    import rosa_soft_b200 as rs
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 50, 4, 6, generator=g)
    h = rs.symbol_health(x, 0.1)
    assert abs(h.positive_fraction - float((x > 0).float().mean())) < 1e-7
    per_bit = (x > 0).float().mean(dim=(0, 1, 2))
    assert abs(h.bit_imbalance - float((2 * (per_bit - 0.5).abs()).mean())) < 1e-7
    assert abs(h.sign_margin_low_quantile - float(torch.quantile(x.abs().reshape(-1), 0.1))) < 1e-6
    routes = torch.tensor([[[0, 1, 0, 2, 4]]])            # [B=1, H=1, T=5]
    lens = torch.tensor([[[0, 1, 0, 3, 2]]])
    info = rs.HardRouteInspection(routes, lens, 3, torch.arange(5))
    d = rs.summarize_hard_routes(info, x, x)
    assert abs(d.hard_nonnull_route_fraction - 0.6) < 1e-7
    assert abs(d.hard_route_lag_mean - ((1 - 1) + (3 - 2) + (4 - 4)) / 3) < 1e-7
    assert abs(d.selected_match_length_mean - 2.0) < 1e-7
    assert abs(d.horizon_hit_fraction - 1 / 3) < 1e-7
    empty = rs.HardRouteInspection(torch.zeros(1, 1, 4, dtype=torch.int64),
                                   torch.zeros(1, 1, 4, dtype=torch.int64), 3, torch.arange(4))
    assert rs.summarize_hard_routes(empty, x, x).hard_route_lag_mean != \
        rs.summarize_hard_routes(empty, x, x).hard_route_lag_mean      # NaN
