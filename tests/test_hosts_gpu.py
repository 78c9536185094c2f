"""End-to-end on small host models: install the operators with the replacement rules, run
forward + backward, and compare the LoRA gradients with the same host run without
compression (exact autograd)."""
import copy

import pytest
import torch

from hyc_lora_b200 import synthetic

pytestmark = pytest.mark.gpu


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def _lora_grads(model):
    return {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.requires_grad and p.grad is not None}


def _train_b(model, seed=3):
    """LoRA-B starts at zero, which makes every LoRA-A gradient zero: give it values."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    for n, p in model.named_parameters():
        if "lora_B" in n:
            p.data.normal_(0, 0.05, generator=g)


@pytest.mark.parametrize("extra,bits,floor", [
    ({}, 8, 0.99), ({}, 4, 0.98),
    (dict(outlier_mode="channel", rotate=256), 8, 0.999), (dict(outlier_mode="channel", rotate=256), 4, 0.98),
    (dict(outlier_mode="channel", group_size=128), 4, 0.98)])
def test_decoder_host_lora_gradients(extra, bits, floor):
    from hyc_lora_b200.hosts.llama import DecoderConfig, DecoderLM
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    cfg = DecoderConfig(hidden=1024, layers=2, heads=8, kv_heads=4, ffn=2816, vocab=512, lora_r=16, base_quant="nf4")
    model = DecoderLM(cfg, seed=1)
    _train_b(model)
    ids = synthetic.token_ids(3, 2, 64, cfg.vocab).cuda()
    exact = copy.deepcopy(model)
    exact(ids).backward()
    want = _lora_grads(exact)
    n = replace_module(model, uniform_config(sub_outlier_bit=bits, sub_outlier_quantize_method="per-channel"), extra)
    # per layer: 7 LoRA-A linears, 2 norms, SiLU, product; plus the final norm
    assert n == cfg.layers * 11 + 1
    for step in range(3):                                 # two calibration calls, then a steady-state call
        model.zero_grad(set_to_none=True)
        loss = model(ids)
        loss.backward()
    got = _lora_grads(model)
    assert set(k.replace(".weight", "") for k in got) == set(k.replace(".weight", "") for k in want)
    assert abs(loss.item() - exact(ids).item()) < 2e-2
    cos = [_cos(got[k], want[k]) for k in want]
    assert min(cos) > floor - 0.03 and sum(cos) / len(cos) > floor, (min(cos), sum(cos) / len(cos))


def test_frozen_nf4_linear_matches_codebook_dequantisation():
    from hyc_lora_b200.hosts import lora
    w = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16) * 0.02
    codes, absmax = lora.nf4_quantize(w)
    got = lora.nf4_dequantize(codes, absmax, w.shape)
    book = lora.nf4_codebook().cuda()
    idx = torch.stack((codes >> 4, codes & 15), dim=1).reshape(-1, 64).long()
    want = (book[idx] * absmax[:, None]).to(torch.bfloat16).reshape(w.shape)
    assert torch.equal(got, want)
    assert (got.float() - w.float()).abs().max() <= 0.16 * w.float().abs().max()
    layer = lora.FrozenLinear(512, 256, "nf4", device="cuda")
    x = torch.randn(4, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    layer(x).sum().backward()
    assert x.grad is not None and not any(p.requires_grad for p in layer.parameters())


def test_encoder_host_runs_with_every_operator_installed():
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    from hyc_lora_b200.hosts.roberta import EncoderClassifier, EncoderConfig
    cfg = EncoderConfig(hidden=768, layers=2, heads=12, ffn=3072, vocab=1000, max_pos=140)
    model = EncoderClassifier(cfg, seed=2)
    _train_b(model)
    ids = synthetic.token_ids(2, 4, 128, cfg.vocab).cuda()
    labels = torch.randint(0, 2, (4,), generator=torch.Generator().manual_seed(1)).cuda()
    exact = copy.deepcopy(model).eval()        # the installed dropout is the identity (p = 0), so compare without dropout
    exact(ids, labels).backward()
    want = _lora_grads(exact)
    # Random-init attention is nearly flat, so a 5 % sparse copy of the probabilities (the reference's
    # preset, which assumes peaked attention) cannot reproduce the softmax gradient; keep 98 % here to
    # test the plumbing of every operator, and 5 % below to check that it still runs.
    n = replace_module(model, uniform_config(sub_outlier_bit=8, sub_outlier_quantize_method="per-channel",
                                             softmax_outlier_ratio=0.98))
    # per layer: 2 LoRA-A (query, value), gemm1, gemm2, softmax, dropout, 2 LayerNorms, GELU; plus the embedding LayerNorm
    assert n == cfg.layers * 9 + 1
    for _ in range(3):
        model.zero_grad(set_to_none=True)
        model(ids, labels).backward()
    got = _lora_grads(model)
    cos = [_cos(got[k], want[k]) for k in want if "lora" in k]
    assert min(cos) > 0.97 and sum(cos) / len(cos) > 0.99, (min(cos), sum(cos) / len(cos))


def test_encoder_host_with_the_reference_preset_sparsity():
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    from hyc_lora_b200.hosts.roberta import EncoderClassifier, EncoderConfig
    cfg = EncoderConfig(hidden=768, layers=1, heads=12, ffn=3072, vocab=1000, max_pos=140)
    model = EncoderClassifier(cfg, seed=4)
    _train_b(model)
    replace_module(model, uniform_config(sub_outlier_bit=4, softmax_outlier_ratio=0.05))
    ids = synthetic.token_ids(2, 4, 128, cfg.vocab).cuda()
    labels = torch.zeros(4, dtype=torch.long, device="cuda")
    for _ in range(3):
        model.zero_grad(set_to_none=True)
        loss = model(ids, labels)
        loss.backward()
    grads = _lora_grads(model)
    assert torch.isfinite(loss) and all(torch.isfinite(g).all() for g in grads.values())


def test_graph_captured_step_matches_eager_step():
    from hyc_lora_b200.hosts.step import build_trainer
    ids = synthetic.token_ids(3, 2, 128, 32000).cuda()
    losses = {}
    for mode in ("eager", "graph"):
        tr = build_trainer("llama2_7b", layers=2, seed=5)
        for _ in range(3):
            tr.step(ids)
        if mode == "graph":
            assert tr.capture(ids)
        out = []
        for _ in range(4):
            out.append(float(tr.step(ids).item()))
        losses[mode] = out
    assert losses["graph"][-1] < losses["graph"][0]                 # it trains
    for a, b in zip(losses["eager"], losses["graph"]):
        assert abs(a - b) < 2e-2 * abs(a)


@pytest.mark.parametrize("case", ["decoder", "decoder_bf16", "decoder_int2", "decoder_rank2", "encoder"])
def test_lora_gradients_match_the_reference_operators(case):
    """LoRA gradients of small hosts with this package's operators (reference mode) against the
    reference's own operator classes: the decoder in fp32, in bf16 at 1 024 channels, at INT2 with 2 %
    outliers and with a rank-2 low-rank part (frozen statistics loaded from the fixture), and the encoder
    with every eager-attention operator.  Bar: cosine >= 0.999 for every adapter matrix.

    Two comparisons.  (1) Against fixtures made on CPU (tests/golden/make_e2e_golden.py), which travel
    everywhere.  (2) When the reference's sources are on this machine, against the same host with the
    reference's classes installed and run on this very device, which takes the CPU-vs-GPU difference of
    the library GEMMs out of the comparison.  That difference matters in bf16 only: there the reference's
    own operators on the GPU reach just 0.9990 against themselves on CPU (activations that differ in their
    last bf16 bit flip quantisation codes, and exact autograd on the two devices already differs at
    0.99995), so the bf16 fixture is held to 0.998 and the bar proper is comparison (2)."""
    import os
    import numpy as np
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    from oracle import ref_loader
    from tests.golden import make_e2e_golden as gold
    c = gold.CASES[case]
    bf16 = c["cfg"]["dtype"] == torch.bfloat16
    fix = np.load(os.path.join(os.path.dirname(gold.__file__), f"e2e_{case}.npz"))
    model = gold.build_host(device="cuda", case=case)
    cfg = uniform_config(softmax_outlier_ratio=c.get("softmax_ratio", 0.05), **c["site"])
    n = replace_module(model, cfg)
    layers = c["cfg"]["layers"]
    assert n == (layers * 11 + 1 if c["kind"] == "decoder" else layers * 9 + 1)
    if c["calibrate"]:
        assert gold.load_calibration(model, fix, "cuda") == n
    from hyc_lora_b200 import packed
    packed.reset_status()
    args = tuple(a.cuda() for a in gold.inputs(case))
    loss = model(*args)
    loss.backward()
    assert abs(loss.item() - float(fix["loss"])) < (2e-2 if bf16 else 1e-3)
    worst, seen = 1.0, 0
    for name, p in model.named_parameters():
        if "grad/" + name in fix.files:
            worst = min(worst, _cos(p.grad.cpu(), torch.from_numpy(fix["grad/" + name])))
            seen += 1
    assert seen == sum(1 for k in fix.files if k.startswith("grad/"))
    assert worst >= (0.998 if bf16 else 0.999), worst
    assert packed.poll_status(wait=True) == 0             # no outlier pool overflowed, no wait gave up

    if ref_loader.load() is None or c["calibrate"]:
        return      # (the calibrated case would need the reference's randomized SVD to repeat on this device)
    ref = gold.build_host(device="cuda", case=case)
    gold._install_reference(ref, case)
    ref(*args).backward()
    want = {k: p.grad for k, p in ref.named_parameters() if p.grad is not None}
    worst = min(_cos(p.grad, want[k]) for k, p in model.named_parameters() if "grad/" + k in fix.files)
    assert worst >= 0.999, worst


@pytest.mark.parametrize("hq,hk,hd,s", [(4, 4, 128, 37), (8, 2, 64, 16)])
def test_rotary_kernel_matches_tensor_ops(hq, hk, hd, s):
    """The fused in-place rotary kernel against the tensor-op formulation (fp32), forward and backward."""
    from hyc_lora_b200.hosts.llama import _rope
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, s, hq, hd, generator=g).to(torch.bfloat16)
    k = torch.randn(2, s, hk, hd, generator=g).to(torch.bfloat16)
    gq, gk = torch.randn(2, s, hq, hd, generator=g), torch.randn(2, s, hk, hd, generator=g)
    # reference: the same function on CPU fp32 tensors takes the tensor-op path
    qr, kr = q.float().requires_grad_(True), k.float().requires_grad_(True)
    yq, yk = _rope(qr.reshape(2, s, hq * hd), kr.reshape(2, s, hk * hd), 10000.0, hq, hk)
    ((yq * gq).sum() + (yk * gk).sum()).backward()
    qd, kd = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    # fresh non-view tensors: the kernel rotates them in place
    zq, zk = _rope((qd * 1).reshape(2, s, hq * hd) + 0, (kd * 1).reshape(2, s, hk * hd) + 0, 10000.0, hq, hk)
    ((zq.float() * gq.cuda()).sum() + (zk.float() * gk.cuda()).sum()).backward()
    for got, want in ((zq, yq), (zk, yk), (qd.grad, qr.grad), (kd.grad, kr.grad)):
        got, want = got.detach().float().cpu(), want.detach().float()
        assert (got - want).abs().max() <= 1e-2 * want.abs().max() + 1e-3
        assert _cos(got, want) > 0.9999


@pytest.mark.parametrize("quant", ["nf4", "bf16"])
def test_input_gradients_summed_along_the_carry(quant):
    """Projections that read one activation hand a carry from one to the next; the gradient that reaches
    the activation must be the sum of every base and LoRA-A input gradient (worked out here with plain
    products in fp32), and the LoRA gradients must not depend on whether a carry was used."""
    from hyc_lora_b200.hosts.lora import LoRALinear
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    torch.manual_seed(5)
    mods = torch.nn.ModuleList(LoRALinear(1024, o, r=16, quant=quant, device="cuda") for o in (1024, 512, 256))
    _train_b(mods)
    assert replace_module(mods, uniform_config(sub_outlier_bit=8), dict(outlier_mode="channel")) == 3
    x0 = torch.randn(2, 64, 1024, device="cuda", dtype=torch.bfloat16)
    gy = [torch.randn(2, 64, m.base_layer.out_features, device="cuda", dtype=torch.bfloat16) for m in mods]

    def run(chained):
        for m in mods:
            m.zero_grad(set_to_none=True)
        x = x0.clone().requires_grad_(True)
        xa = x * 1.0                                   # a non-leaf activation, as in a host
        carry, ys = xa, []
        for m in mods:
            if chained:
                y, carry = m(xa, carry=carry)
            else:
                y = m(xa)
            ys.append(y)
        torch.autograd.backward(ys, gy)
        return x.grad.float(), [m.lora_A.weight.grad.clone() for m in mods], [m.lora_B.weight.grad.clone() for m in mods]

    for _ in range(3):                                 # calibration calls, then the steady state
        gx_c, ga_c, gb_c = run(True)
    gx_u, ga_u, gb_u = run(False)
    want = torch.zeros_like(gx_c)
    for m, g in zip(mods, gy):
        w = m.base_layer.dense_weight().float()
        gh = (g.float().reshape(-1, g.shape[-1]) @ m.lora_B.weight.float()) * m.scaling
        want += (g.float().reshape(-1, g.shape[-1]) @ w + gh.to(torch.bfloat16).float() @ m.lora_A.weight.float()).view(want.shape)
    scale = want.abs().max().item()
    assert (gx_c - want).abs().max().item() < 2e-2 * scale
    assert (gx_u - want).abs().max().item() < 3e-2 * scale
    for a, b in zip(ga_c + gb_c, ga_u + gb_u):
        assert torch.equal(a, b)


def test_gradients_added_into_the_owner_s_buffer_match_the_engine_s_accumulation():
    """Parameters that carry a ``hyc_grad_sink`` (what ``FlatGradSync(fused_accumulate=True)`` sets) get their
    gradients added into ``param.grad`` by the producing kernels; the result must be what the autograd engine's own
    accumulation gives, the sink must be called once per parameter and backward pass, and a second pass must add."""
    from hyc_lora_b200.ddp import FlatGradSync
    from hyc_lora_b200.hosts.lora import LoRALinear, lora_parameters
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    torch.manual_seed(11)
    mods = torch.nn.ModuleList(LoRALinear(1024, o, r=16, quant="bf16", device="cuda") for o in (1024, 256))
    _train_b(mods)
    assert replace_module(mods, uniform_config(sub_outlier_bit=4), dict(outlier_mode="channel", rotate=256)) == 2
    x0 = torch.randn(2, 64, 1024, device="cuda", dtype=torch.bfloat16)
    gy = [torch.randn(2, 64, m.base_layer.out_features, device="cuda", dtype=torch.bfloat16) for m in mods]

    def backward_pass():
        x = x0.clone().requires_grad_(True)
        torch.autograd.backward([m(x) for m in mods], gy)

    for _ in range(3):                                 # calibration calls, then the steady state
        mods.zero_grad(set_to_none=True)
        backward_pass()
    params = lora_parameters(mods)
    want = [p.grad.clone() for p in params]
    sync = FlatGradSync(params, fused_accumulate=True)   # every .grad is now a view of the (zeroed) flat buffer
    calls = []
    for i, p in enumerate(params):
        inner = p.hyc_grad_sink
        p.hyc_grad_sink = lambda i=i, inner=inner: (calls.append(i), inner())[1]
    backward_pass()
    assert sorted(calls) == list(range(len(params)))
    for p, w in zip(params, want):
        assert p.grad.data_ptr() >= sync.flat.data_ptr() and torch.equal(p.grad, w)
    backward_pass()                                     # a second pass adds (one rounding of the fp32 sum)
    for p, w in zip(params, want):
        assert (p.grad.float() - 2 * w.float()).abs().max() <= 2e-2 * w.float().abs().max()
    assert len(calls) == 2 * len(params)
