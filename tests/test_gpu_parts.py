"""Each part of a layer alone against its plain counterpart: norm, position encoding, mixer
(attention), feed-forward, block, embedding and output head.  The parts are taken out of a loaded
tiny model and called directly; only the step context (page tables, positions) comes from the
runner."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def close(got, ref, dtype, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    tol = 1e-5 * max(1.0, ref.abs().max().item()) if dtype == "float32" else 0.03 * max(ref.abs().max().item(), 1e-3)
    d = (got - ref).abs().max().item()
    assert torch.isfinite(got).all() and d <= tol, f"{what}: max diff {d:.3e} > {tol:.3e}"


@pytest.fixture(scope="module", params=[(n, d) for n in ("tiny-a", "tiny-b") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, model_folders):
    name, dtype = request.param
    folder = model_folders(name, dtype)
    r = helpers.Replayer(folder, dtype, 256, helpers.TINY[name]["block_size"])
    cfg, w = P.read_model_folder(folder)
    return dict(name=name, dtype=dtype, r=r, cfg=cfg, w=w, sizes=P.sizes_from_config(cfg),
                storage=None if dtype == "float32" else torch.bfloat16)


def step_context(r, n, start=0):
    """Context of one request computing positions [start, start + n); pages are taken as needed."""
    seq = r.core.Sequence()
    seq.id = 77
    seq.state_slot = r.slots.take()
    r.kv.admit(seq)
    seq.extend_tokens([1] * (start + n))
    assert r.kv.ensure(seq, start + n)
    layout = r.runner.build([(seq, start, n, [])])
    r.runner.upload(layout)
    return seq, r.runner.context(layout)


def finish(r, seq):
    torch.cuda.synchronize()
    r.kv.release(seq)
    r.slots.give_back(seq.state_slot)


def test_norm_part(setup):
    s = setup
    spec, c = s["r"].spec, s["sizes"]
    norm = spec.blocks[0].norm1
    assert norm.eps == c["eps"] and norm.hidden == c["H"]
    x = torch.randn(11, c["H"]) * 2
    pend = torch.randn(11, c["H"]).to(DT[s["dtype"]])
    xd = x.clone().cuda()
    out = torch.empty(11, c["H"], dtype=DT[s["dtype"]], device="cuda")
    norm.forward(xd, pend.cuda(), out)
    x_new = x.double() + pend.double()
    close(xd, x_new, "float32", "residual")
    close(out, P.rmsnorm(x_new, s["w"]["model.layers.0.input_layernorm.weight"], c["eps"], s["storage"]),
          s["dtype"], "norm")


def test_position_encoding_part(setup):
    s = setup
    c = s["sizes"]
    pos = s["r"].spec.blocks[0].mixer.position
    assert pos.rotary_dim == c["hd"] and not pos.interleaved and pos.theta == c["theta"]
    j = torch.arange(c["hd"] // 2, dtype=torch.float64)
    want = 1.0 / torch.pow(torch.tensor(c["theta"], dtype=torch.float64), 2.0 * j / c["hd"])
    assert torch.allclose(pos.inv_freq.cpu().double(), want, rtol=1e-6)


def test_mixer_part(setup):
    s = setup
    c, w = s["sizes"], s["w"]
    mixer = s["r"].spec.blocks[1].mixer
    n = 70
    seq, ctx = step_context(s["r"], n)
    h = torch.randn(n, c["H"]).to(DT[s["dtype"]])
    got = mixer.forward(h.cuda(), ctx, s["r"].runner.pools.sites[1])
    p = "model.layers.1.self_attn."
    ref = P.attention_block(h.double(), w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"],
                            w[p + "o_proj.weight"], torch.arange(n), c, None, s["storage"])
    close(got, ref, s["dtype"], "attention mixer")
    finish(s["r"], seq)


def test_feed_forward_part(setup):
    s = setup
    c, w = s["sizes"], s["w"]
    ffn = s["r"].spec.blocks[0].ffn
    seq, ctx = step_context(s["r"], 9)
    h = torch.randn(9, c["H"]).to(DT[s["dtype"]])
    got = ffn.forward(h.cuda(), ctx)
    p = "model.layers.0.mlp."
    ref = P.gated_mlp(h.double(), w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"],
                      s["storage"])
    close(got, ref, s["dtype"], "gated MLP")
    finish(s["r"], seq)


def test_block_part(setup):
    s = setup
    c, w = s["sizes"], s["w"]
    block = s["r"].spec.blocks[0]
    n = 40
    seq, ctx = step_context(s["r"], n)
    x = torch.randn(n, c["H"])
    xd = x.clone().cuda()
    pending = block.forward(xd, None, ctx, s["r"].runner.pools.sites[0])
    p = "model.layers.0."
    xr = x.double()
    hh = P.rmsnorm(xr, w[p + "input_layernorm.weight"], c["eps"], s["storage"])
    xr = xr + P.attention_block(hh, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                                w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"],
                                torch.arange(n), c, None, s["storage"])
    hh = P.rmsnorm(xr, w[p + "post_attention_layernorm.weight"], c["eps"], s["storage"])
    mlp = P.gated_mlp(hh, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                      w[p + "mlp.down_proj.weight"], s["storage"])
    close(xd, xr, s["dtype"], "residual after the mixer")          # the MLP output is still pending
    close(pending, mlp, s["dtype"], "pending MLP output")
    finish(s["r"], seq)


def test_embedding_and_head_parts(setup):
    s = setup
    c, w = s["sizes"], s["w"]
    spec = s["r"].spec
    seq, ctx = step_context(s["r"], 5)
    x = spec.embedding.forward(ctx)
    assert torch.equal(x.cpu().double(), w["model.embed_tokens.weight"][[1] * 5])
    h = torch.randn(5, c["H"]).to(DT[s["dtype"]])
    logits = spec.lm_head.forward(h.cuda(), ctx)
    lm = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    assert logits.dtype == torch.float32
    close(logits, h.double() @ lm.T, "float32" if s["dtype"] == "float32" else "bfloat16", "output head")
    finish(s["r"], seq)


def test_parts_are_chosen_by_name_from_registries():
    from kvcm.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
    assert "attention" in MIXERS.names() and "gated_mlp" in FEED_FORWARDS.names()
    assert "rmsnorm" in NORMS.names() and {"rope", "none"} <= set(POSITION_ENCODINGS.names())
    assert "pre_norm" in BLOCKS.names()
    with pytest.raises(KeyError):
        MIXERS.get("no-such-mixer")
    with pytest.raises(ValueError):
        FEED_FORWARDS.build("gated_mlp", hidden=8, intermediate=8, activation="gelu")
