"""The other reference-facing surfaces on the GPU: the `onebit_sparse_cuda` torch extension (both
argument orders the reference uses), the drop-in `onebit_sparse_mul` import name, and the `a.out`
CLI with the reference's flags and output lines."""
import os
import re
import subprocess

import numpy as np
import pytest
import torch

import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def problem():
    rng = np.random.default_rng(77)
    m, k, n = 256, 512, 40
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, oracle.META_PYTHON)
    B = helpers.make_tokens(rng, k, n, "int")
    want, _ = oracle.gemm(bits, meta, oracle.META_PYTHON, B, m)
    want_scaled, _ = oracle.gemm(bits, meta, oracle.META_PYTHON, B, m, scale=scale)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return dict(m=m, k=k, n=n, A=t(bits), meta=t(meta.view(np.int16)), B=t(B), scale=t(scale), want=want, want_scaled=want_scaled)


def test_torch_extension_both_argument_orders(problem):
    from onebitsparsemul_b200 import build
    build.build_torch_extension()
    import onebit_sparse_cuda
    p = problem
    C = torch.zeros((p["m"], p["n"]), dtype=torch.float32, device="cuda")
    onebit_sparse_cuda.onebit_mul(p["A"], p["B"], p["meta"], C)              # the reference's C++ order
    assert (C.cpu().numpy() == p["want"]).all()
    C.zero_()
    onebit_sparse_cuda.onebit_mul(p["A"], p["B"], C, p["meta"])              # the reference's Python order
    assert (C.cpu().numpy() == p["want"]).all()
    C16 = torch.zeros((p["m"], p["n"]), dtype=torch.float16, device="cuda")
    onebit_sparse_cuda.onebit_mul(p["A"], p["B"], p["meta"], C16, p["scale"])
    ok, worst = helpers.row_tolerance_ok(C16.cpu().numpy(), p["want_scaled"])
    assert ok, worst
    with pytest.raises(RuntimeError):
        onebit_sparse_cuda.onebit_mul(p["A"], p["B"], p["meta"], torch.zeros((p["m"], p["n"] + 1), device="cuda"))
    with pytest.raises(RuntimeError):
        onebit_sparse_cuda.onebit_mul(p["A"], p["B"].cpu(), p["meta"], C)


def test_reference_import_name(problem):
    import onebit_sparse_mul as ref_name
    p = problem
    C = ref_name.cuda_binary_mul(p["A"], p["B"], p["meta"])
    assert C.dtype == torch.float32 and C.is_cuda and (C.cpu().numpy() == p["want"]).all()
    C2 = torch.empty_like(C)
    assert ref_name.cuda_binary_mul_(p["A"], p["B"], C2, p["meta"]) is C2 and (C2 == C).all()
    layer = ref_name.BinaryLinear_2_4(128, 128)
    assert layer.vaild is False and tuple(layer.packed_binary_sparse.shape) == (64, 16) and tuple(layer.meta.shape) == (128, 8)


def run_cli(*args):
    exe = os.path.join(ROOT, "a.out")
    if not os.path.exists(exe):
        from onebitsparsemul_b200 import build
        build.build_cli()
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=300)


def test_cli_reference_flags_and_output_lines():
    r = run_cli("--a_rows=512", "--n=512", "--a_cols=512", "--reference-check=true", "--iterations=5",
                "--alpha=1", "--beta=0", "--a_ell_num_columns=512", "--a_ell_blocksize=16", "--a_base=0")
    lines = r.stdout.strip().splitlines()
    assert r.returncode == 0, r.stdout + r.stderr
    assert re.fullmatch(r"Runtime: [0-9.e+-]+ ms", lines[0]) and re.fullmatch(r" GFLOPs: [0-9.e+-]+", lines[1])
    assert lines[2] == "Passed"
    # the reference's degenerate fill through the reference's own entry point, exact check
    r = run_cli("--a_rows=256", "--n=64", "--a_cols=256", "--dist=reference", "--stateless=true", "--reference-check=true", "--iterations=2")
    assert r.returncode == 0 and r.stdout.strip().endswith("Passed")
    # decode shape, fp16 output with scale, JSON mode
    r = run_cli("--a_rows=4096", "--n=4", "--a_cols=4096", "--out=fp16", "--scale=true", "--reference-check=true", "--json")
    assert r.returncode == 0 and '"passed": true' in r.stdout
    assert "--a_rows" in run_cli("--help").stdout


def test_model_replace_flow_and_state_dict_round_trip():
    """The step above the path (reference: tests/python/test_model_replace.py:22-44) on a synthetic
    Llama-shaped MLP block: swap nn.Linear layers, run tokens through, save and reload."""
    import torch.nn as nn

    import onebitsparsemul_b200 as ob

    torch.manual_seed(0)

    class Block(nn.Module):
        def __init__(self, d=256, f=512):
            super().__init__()
            self.gate, self.up, self.down = nn.Linear(d, f, bias=False), nn.Linear(d, f, bias=True), nn.Linear(f, d, bias=False)
            self.lm_head = nn.Linear(d, 384, bias=False)
            self.odd = nn.Linear(d, 100)                                   # not a multiple of 128: left alone

        def forward(self, x):
            return self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))

    model = Block().cuda().half()
    x = torch.randn(3, 5, 256, device="cuda", dtype=torch.float16)
    # what the replaced model should compute: sign(w) * mask * scale in place of w
    def quantised(lin):
        w = lin.weight.detach()
        mask = ob.mask_creator(w)
        scale = ((w.float().abs() * mask).sum(1) / mask.sum(1)).half()
        return (torch.sign(w.float()) * mask * scale.float()[:, None]).half()
    ref = Block().cuda().half()
    ref.load_state_dict(model.state_dict())
    for name in ("gate", "up", "down"):
        getattr(ref, name).weight.data = quantised(getattr(model, name))
    want = ref(x)

    n = ob.replace_linear_layers(model)
    assert n == 3 and isinstance(model.gate, ob.BinaryLinear_2_4) and isinstance(model.lm_head, nn.Linear) and isinstance(model.odd, nn.Linear)
    got = model(x)
    assert got.shape == want.shape and got.dtype == torch.float16
    assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2 * want.float().abs().max().item())

    # checkpoint / resume: the packed tensors travel in the state dict
    state = {k: v.cpu() for k, v in model.state_dict().items()}
    assert {"gate.bits_tile", "gate.meta_tile", "gate.scale", "gate.packed_binary_sparse", "gate.meta", "up.bias"} <= set(state)
    fresh = Block().half()
    fresh.gate, fresh.up, fresh.down = ob.BinaryLinear_2_4(256, 512), ob.BinaryLinear_2_4(256, 512, bias=True), ob.BinaryLinear_2_4(512, 256)
    for m_ in (fresh.gate, fresh.up, fresh.down):
        m_.forward = m_.forward_tokens
    fresh.load_state_dict(state)
    fresh = fresh.cuda()
    assert fresh.gate.vaild and torch.equal(fresh(x), got)


@pytest.mark.parametrize("m,n,k", [(256, 64, 256), (512, 4096, 1024), (1024, 2056, 512)])
def test_host_buffer_entry_point_equals_device_path(m, n, k):
    """onebit_matmul_packed_host (pinned host tokens in, pinned host result out, pipelined copies) gives
    the bits the device-resident call gives, also when the last column panel is ragged (integer tokens:
    a narrow last panel may run on another kernel, whose summation order differs)."""
    import onebitsparsemul_b200 as ob
    rng = np.random.default_rng(m + n)
    dense, scale = helpers.make_weights(rng, m, k)
    pw = ob.pack_weight(torch.from_numpy(dense), scale=torch.from_numpy(scale), apply_mask=False)
    Bh = torch.from_numpy(helpers.make_tokens(rng, k, n, "int")).pin_memory()
    for dtype in (torch.float16, torch.float32):
        want = ob.matmul_packed(pw, Bh.cuda(), out_dtype=dtype)
        for _ in range(2):                                   # twice: slot reuse across calls
            Ch = torch.full((m, n), float("nan"), dtype=dtype).pin_memory()
            ob.matmul_packed_host(pw, Bh, Ch)
            torch.cuda.synchronize()
            assert torch.equal(Ch, want.cpu())
    with pytest.raises(ValueError):
        ob.matmul_packed_host(pw, torch.zeros((k, n), dtype=torch.float16))     # not pinned


def test_llama_shaped_stack_replace_and_graph_decode_loop():
    """The reference's model-replace flow (tests/python/test_model_replace.py:22-44) on a Llama-shaped stack, and the
    decode loop a model runs: one token at a time through a CUDA graph. The graph must give the bits of the eager
    run, and the replaced stack must equal the same stack evaluated with the dequantised weights."""
    import onebitsparsemul_b200 as ob
    from onebitsparsemul_b200.decode_loop import GraphedDecoder, LlamaShapedStack, measure_decode
    hidden, inter = 512, 1408
    stack = LlamaShapedStack(blocks=2, hidden=hidden, intermediate=inter, device="cuda", seed=5)
    ref = LlamaShapedStack(blocks=2, hidden=hidden, intermediate=inter, device="cuda", seed=5)
    assert ob.replace_linear_layers(stack) == 14
    # reference stack: the same layers with the dequantised one-bit weights as dense fp32 matrices
    for blk, rblk in zip(stack.blocks, ref.blocks):
        for name in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
            packed = getattr(blk, name)
            dense = torch.empty((packed.outfeatures, packed.infeatures), dtype=torch.float16, device="cuda")
            _lib.check(_lib.load().onebit_unpack_to_dense(packed.bits_tile.data_ptr(), packed.meta_tile.data_ptr(), packed.scale.data_ptr(),
                                                          packed.outfeatures, packed.infeatures, dense.data_ptr(), None))
            getattr(rblk, name).weight.data = dense
    torch.manual_seed(3)
    ref = ref.float()
    for tokens in (1, 4, 40):
        x = torch.randn((tokens, hidden), device="cuda").to(torch.float16)
        with torch.no_grad():
            eager = stack(x)
            want = ref(x.float())
        assert torch.isfinite(eager).all()
        err = (eager.float() - want.float()).abs().max().item()
        assert err <= 2e-2 * want.float().abs().max().item() + 1e-3, err
        dec = GraphedDecoder(stack, tokens, hidden)
        for _ in range(3):                                      # replays are repeatable and equal the eager run
            assert torch.equal(dec.step(x), eager)
        _lib.check(_lib.load().onebit_check_device_status())
    m = measure_decode(stack, hidden, tokens=1, steps=5)
    assert m["linear_layers"] == 14 and m["us_per_step"] > 0
    # q/k/v and gate/up as one layer each: the same weights stacked give the same activations (every output row is
    # its own dot product, whatever matrix it sits in; the K split and with it the fp32 summation order may differ)
    fused = LlamaShapedStack(blocks=2, hidden=hidden, intermediate=inter, device="cuda", seed=5, fused=True)
    plain = LlamaShapedStack(blocks=2, hidden=hidden, intermediate=inter, device="cuda", seed=5)
    with torch.no_grad():
        for fb, pb in zip(fused.blocks, plain.blocks):
            fb.qkv_proj.weight.copy_(torch.cat([pb.q_proj.weight, pb.k_proj.weight, pb.v_proj.weight]))
            fb.gate_up_proj.weight.copy_(torch.cat([pb.gate_proj.weight, pb.up_proj.weight]))
            fb.o_proj.weight.copy_(pb.o_proj.weight)
            fb.down_proj.weight.copy_(pb.down_proj.weight)
    assert ob.replace_linear_layers(fused) == 8 and ob.replace_linear_layers(plain) == 14
    x = torch.randn((4, hidden), device="cuda").to(torch.float16)
    with torch.no_grad():
        yf, yp = fused(x).float(), plain(x).float()
    assert (yf - yp).abs().max().item() <= 1e-2 * yp.abs().max().item() + 1e-3


def test_pitched_copy_helper_moves_a_column_panel_both_ways():
    """onebit_copy_2d_async: a column panel of a row-major host matrix to a contiguous device buffer and back into
    another host matrix (the building block of the row-sharded host path)."""
    lib = _lib.load()
    rows, cols, c0, w = 300, 1000, 128, 256
    src = (torch.arange(rows * cols, dtype=torch.int32) % 2048 + 1).to(torch.float16).reshape(rows, cols).pin_memory()
    dst = torch.zeros((rows, cols), dtype=torch.float16).pin_memory()
    panel = torch.empty((rows, w), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.onebit_copy_2d_async(panel.data_ptr(), w * 2, src.data_ptr() + c0 * 2, cols * 2, w * 2, rows, stream))
    _lib.check(lib.onebit_copy_2d_async(dst.data_ptr() + c0 * 2, cols * 2, panel.data_ptr(), w * 2, w * 2, rows, stream))
    torch.cuda.synchronize()
    assert torch.equal(panel.cpu(), src[:, c0:c0 + w])
    assert torch.equal(dst[:, c0:c0 + w], src[:, c0:c0 + w])
    assert not dst[:, :c0].any() and not dst[:, c0 + w:].any()
    # a pitch smaller than a row is refused, nothing is copied
    assert lib.onebit_copy_2d_async(panel.data_ptr(), w, src.data_ptr(), cols * 2, w * 2, rows, stream) == 5    # ONEBIT_ERR_ARG
