"""The Fobanex design against a plain float64 implementation (``plain_fobanex``): every
mechanism alone on made inputs, then whole models of several shapes through the step function
(whole prompts, decoding, portions, mixed batches, replay, generation)."""
from __future__ import annotations

import json
import math
from types import SimpleNamespace

import pytest
import torch

import plain_fobanex as pf
import trace_util as tu
from conftest import random_tokens, read_folder

DTYPES = ["float32", "bfloat16"]


# ---------------------------------------------------------------------- configurations
def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _att(heads, kv, dim, vdim, scale, rot):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim,
                                           "scale": scale, "rot": rot}}


def _att2(heads, kv, dim, scale, rot):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                                             "scale": scale, "rot": rot}}


def _lat(heads, dim, rot_dim, vdim, rank, q_rank, scale, base, kv_from=None, scaling=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
          "scale": scale, "rot": _rot(rot_dim, base, scaling)}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx}


def _moe(ff, experts, top, limit, groups=None, scale=None):
    ro = {"experts": experts, "top": top}
    if groups:
        ro["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        ro["scale"] = scale
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": ro}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _model(vocab, width, eps, emb_scale, layers):
    cfg = {"architecture": "Fobanex", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    return cfg


# heads of 32 (the tensor-core kernels' smallest), a latent of 64 + 16 (the tensor-core latent
# kernel), a scaled rotation on a quarter of a head and a rotation of the whole head, two layers
# that read the rows of a third, a last layer without a feed-forward
FB_A = _model(211, 96, 1e-5, 12.0, [
    (_att(4, 2, 32, 32, 0.2, _rot(8, 10000.0, (4.0, 64, 16.0, 1.0))), _dense(80)),
    (_lat(4, 32, 16, 32, 64, 40, 0.15, 10000.0), _moe(40, 8, 2, 2.0, (4, 2), 1.5)),
    (_att2(4, 1, 32, 0.18, _rot(32, 500.0)), _moe(40, 8, 2, 2.0, (4, 2), 1.5)),
    (_lat(4, 32, 16, 32, 64, 24, 0.15, 10000.0, kv_from=1), _moe(40, 8, 3, 2.0, (2, 1), 0.7)),
    (_lat(2, 16, 16, 48, 64, 40, 0.2, 10000.0, kv_from=1), None),
])
# a width that is no multiple of 8, heads of 10, values wider than keys, a latent of 20 + 6, no
# embedding scale, a router without groups and without a scale, groups of one expert of which all
# stay, a reader with other heads and sizes than the layer it reads, one query head a KV head
FB_B = _model(131, 50, 2e-6, None, [
    (_lat(2, 10, 6, 12, 20, 7, 0.3, 77.0), _moe(12, 6, 3, 1.0)),
    (_att(3, 3, 10, 14, 0.4, _rot(2, 300.0)), None),
    (_att2(5, 1, 10, 0.3, _rot(10, 1000.0, (2.0, 40, 8.0, 2.0))), _moe(12, 6, 2, 3.0, (6, 6), 2.0)),
    (_lat(3, 8, 6, 6, 20, 9, 0.35, 77.0, kv_from=0), _moe(12, 6, 1, 1.0, (3, 1))),
])
# heads of 64 (attention, keys as values) and a latent of 96 + 32 under heads of 32 with values
# of 64; every expert chosen; one expert a token; a scaled rotation of a latent's shared part
FB_C = _model(180, 128, 1e-5, 0.5, [
    (_att2(2, 2, 64, 0.125, _rot(16, 1000000.0, (8.0, 128, 32.0, 1.0))), _moe(48, 4, 4, 5.0, (2, 2), 0.5)),
    (_att(8, 2, 64, 64, 0.11, _rot(64, 10000.0)), _dense(64)),
    (_lat(4, 32, 32, 64, 96, 128, 0.12, 5000.0, scaling=(4.0, 32, 8.0, 1.0)), _moe(48, 4, 1, 5.0, (2, 1), 1.0)),
])
FB_CONFIGS = {"fb_a": FB_A, "fb_b": FB_B, "fb_c": FB_C}
FB_SEEDS = {"fb_a": 3, "fb_b": 4, "fb_c": 5}
FB_ALONE = {
    "attention_only": _model(97, 64, 1e-5, 3.0, [(_att(4, 2, 16, 16, 0.3, _rot(8, 1000.0)), None)]),
    "key_value_attention_only": _model(97, 64, 1e-5, 3.0, [(_att2(4, 2, 16, 0.3, _rot(6, 1000.0)), None)]),
    "latent_only": _model(97, 64, 1e-5, 3.0, [(_lat(4, 16, 8, 16, 32, 24, 0.3, 1000.0), None)]),
    "latent_borrowed": _model(97, 64, 1e-5, 3.0, [(_lat(4, 16, 8, 16, 32, 24, 0.3, 1000.0), None),
                                                  (_lat(2, 8, 8, 24, 32, 16, 0.3, 1000.0, kv_from=0), None)]),
    "feed_forwards": _model(97, 64, 1e-5, 3.0, [(_att(2, 1, 16, 16, 0.3, _rot(4, 1000.0)), _dense(40)),
                                                (_att(2, 1, 16, 16, 0.3, _rot(4, 1000.0)),
                                                 _moe(24, 9, 2, 1.5, (3, 2), 1.25))]),
}


def _sharpen(cfg, weights, spread=3.0, out=5.0):
    """Random matrices of a small scale give nearly flat attention and mixers that hardly move
    the stream, under which a wrong key would hide.  Scale what the scores grow with (the q and
    k norm weights where the norm runs over the projections, the q and k or the up-projections
    elsewhere) so that a query's scores spread by about ``spread``, and the output projections
    by ``out``."""
    w = {k: v.clone() for k, v in weights.items()}
    std, width = 0.02, cfg["width"]
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.mix.", layer["mixer"]
        want = math.sqrt(spread / (mx["scale"] * math.sqrt(mx["dim"])))      # size of a q and of a k value
        if layer["type"] == "attention":
            w[p + "q.norm"] *= want
            w[p + "k.norm"] *= want
        elif layer["type"] == "attention_2":
            w[p + "q"] *= want / (std * math.sqrt(width))
            w[p + "k"] *= want / (std * math.sqrt(width))
        else:
            w[p + "uq"] *= want / (std * math.sqrt(mx["q_rank"]))
            w[p + "uk"] *= want / (std * math.sqrt(mx["kv_rank"]))
        if p + "g" in w:
            w[p + "g"] *= 20.0                       # gates away from one half
        w[p + "o"] *= out
    return w


def _wide_router_margins(cfg, weights):
    """Make every routed layer's choice a matter of the token id with margins far beyond
    rounding, so that bfloat16 and float64 choose alike, groups included: channels 0..E-1 of
    the embedding hold a code in which every expert has a level of its own (a rotation of
    E, E - 1, ..., 1 by the token id); nothing writes to those channels, so the stream keeps the
    code; the norm passes them with weight 1; router row e of layer i reads the channels c with
    (c + i) % experts == e."""
    w = {k: v.clone() for k, v in weights.items()}
    routed = [l["mlp"] for l in cfg["layers"] if l.get("mlp") and l["mlp"]["kind"] == "moe"]
    if not routed:
        return w
    E = max(ml["router"]["experts"] for ml in routed)
    assert cfg["width"] > E
    scale = cfg.get("embedding", {}).get("scale", 1.0)
    for tok in range(cfg["vocab"]):
        for c in range(E):
            w["embed"][tok, c] = (1.0 + 0.5 * ((c + 5 * tok) % E)) / scale
    for i, layer in enumerate(cfg["layers"]):
        w[f"l{i}.mix.o"][:E, :] = 0.0
        w[f"l{i}.norm1"][:E] = 1.0
        ml = layer.get("mlp")
        if not ml:
            continue
        if ml["kind"] == "dense":
            w[f"l{i}.mlp.down"][:E, :] = 0.0
            w[f"l{i}.mlp.down.b"][:E] = 0.0
            continue
        n_out = ml["router"]["experts"]
        for e in range(n_out):
            w[f"l{i}.mlp.e{e}.down"][:E, :] = 0.0
        r = w[f"l{i}.mlp.router"]
        r[:, :] = 0.0
        for c in range(n_out):                 # one channel an expert: every logit a level of its own
            r[(c + i) % n_out, c] = 1.0
    w["final.norm"][:E] = 0.05
    return w


@pytest.fixture(scope="module")
def fb_folders(tmp_path_factory):
    """Model folders with random weights, sharpened attention and routers with margins;
    ``config.json`` is then written WITHOUT the ranks of the query latents, which a reader has
    to take from the tensors' shapes."""
    from safetensors.torch import save_file
    from helios_b200.weights import write_model_folder

    out = {}
    base = tmp_path_factory.mktemp("fobanex")
    for name, cfg in {**FB_CONFIGS, **FB_ALONE}.items():
        folder = write_model_folder(base / name, cfg, FB_SEEDS.get(name, 9))
        _cfg, weights = read_folder(folder)
        save_file(_wide_router_margins(cfg, _sharpen(cfg, weights)), str(folder / "model.safetensors"))
        lean = json.loads(json.dumps(cfg))
        for layer in lean["layers"]:
            layer["mixer"].pop("q_rank", None)
        (folder / "config.json").write_text(json.dumps(lean))
        out[name] = folder
    return out


def _bf16(weights):
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v.float()) for k, v in weights.items()}


def _f64(weights):
    return {k: v.double() for k, v in weights.items()}


def _plain(cfg, weights, dtype, requests):
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    return {rid: pf.forward(cfg, w, toks)[0] for rid, toks in requests.items()}


def _core(folder, dtype, max_tokens, page_size=16, max_slots=4, graphs=True):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype=dtype)
    return EngineCore(model, page_size=page_size, num_pages=-(-max_tokens // page_size),
                      max_slots=max_slots, poison_cache=float("nan"), use_cuda_graphs=graphs)


def _requests(cfg, lengths, seed):
    return {f"q{i}": random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


# ====================================================================== without a GPU
def test_configuration_is_read_layer_by_layer_and_faults_name_the_key():
    from helios_b200.config import ConfigError
    from helios_b200.config.fobanex_config import (DenseFfnConfig, FobanexConfig, GroupedRouterFfnConfig,
                                                   KeyValueAttentionConfig, QueryLatentAttentionConfig,
                                                   RowNormAttentionConfig)

    cfg = FobanexConfig.from_json(FB_A)
    assert [type(l.mixer) for l in cfg.layers] == [RowNormAttentionConfig, QueryLatentAttentionConfig,
                                                   KeyValueAttentionConfig, QueryLatentAttentionConfig,
                                                   QueryLatentAttentionConfig]
    assert cfg.embedding_scale == 12.0 and cfg.layers[4].mlp is None and isinstance(cfg.layers[0].mlp, DenseFfnConfig)
    assert cfg.layers[0].mixer.rot.scaling.factor == 4.0 and cfg.layers[2].mixer.rot.scaling is None
    assert cfg.layers[3].mixer.kv_from == 1 and cfg.layers[1].mixer.kv_from is None
    ml = cfg.layers[3].mlp
    assert isinstance(ml, GroupedRouterFfnConfig) and (ml.group_count, ml.group_keep, ml.top, ml.scale) == (2, 1, 3, 0.7)
    b = FobanexConfig.from_json(FB_B)
    assert b.embedding_scale == 1.0 and (b.layers[0].mlp.group_count, b.layers[0].mlp.scale) == (1, 1.0)
    for path, value, word in [(("layers", 0, "mixer", "rot", "dims"), 7, "dims"),
                              (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 2, "mixer", "vdim"), 8, "vdim"),
                              (("layers", 1, "mlp", "router", "top"), 5, "top"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups"),
                              (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
                              (("layers", 3, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 3, "mixer", "kv_rank"), 32, "kv_from"),
                              (("layers", 1, "mlp", "expert", "limit"), None, "limit"),
                              (("layers", 0, "type"), "conv", "type"),
                              (("norm",), {}, "eps")]:
        bad = json.loads(json.dumps(FB_A))
        at = bad
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            FobanexConfig.from_json(bad)


def test_plan_names_every_tensor_and_shares_the_borrowed_cache():
    from helios_b200.cache.manager import cache_groups_of
    from helios_b200.config.fobanex_config import FobanexConfig
    from helios_b200.models import build_fobanex_plan
    from helios_b200.weights.loader import expected_tensors

    plan = build_fobanex_plan(FobanexConfig.from_json(FB_A))
    names = expected_tensors(plan)
    for name in ["embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.v", "l0.mix.q.norm", "l0.mix.k.norm",
                 "l0.mlp.gate.b", "l0.mlp.down.b", "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv",
                 "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.g", "l1.mlp.router", "l1.mlp.e7.down",
                 "l2.mix.g", "l2.mix.k", "l3.mix.dq", "l3.mix.uk", "l4.mix.g"]:
        assert name in names, name
    for name in ["l0.mix.g", "l0.norm2", "l2.mix.v", "l2.mix.q.norm", "l3.mix.dkv", "l3.mix.dkv.norm", "l4.mix.dkv",
                 "l1.mix.q", "l4.mlp.router", "l1.mlp.router.b", "l1.mlp.e8.up", "l1.mlp.gate.b"]:
        assert name not in names, name
    assert names["l0.mix.q.norm"][2].shape == (4 * 32,) and names["l0.mix.k.norm"][2].shape == (2 * 32,)
    assert names["l1.mix.uq"][2].shape == (4 * 48, 40) and names["l1.mix.dkv"][2].shape == (64 + 16, 96)
    assert names["l4.mix.uv"][2].shape == (2 * 48, 64) and names["l2.mix.g"][2].shape == (4 * 32, 96)
    assert [(r.layer, r.cache, r.writes_cache) for r in plan.schedule] == \
        [(0, None, True), (1, None, True), (2, None, True), (3, 1, False), (4, 1, False)]
    specs, where = cache_groups_of(plan)
    assert sorted(where) == [0, 1, 2]
    assert {(s.planes, s.num_kv_heads, s.head_dim) for s in specs} == {(2, 2, 32), (1, 1, 80), (2, 1, 32)}


def test_toy_model_of_the_design_from_the_command_line(tmp_path, capsys):
    from helios_b200 import cli

    assert cli.main(["make-toy-model", "--arch", "fobanex", "--out", str(tmp_path / "toy"), "--layers", "5",
                     "--hidden", "64", "--heads", "4", "--kv-heads", "2"]) == 0
    assert cli.main(["info", "--model", str(tmp_path / "toy")]) == 0
    text = capsys.readouterr().out
    assert "Fobanex" in text and "LatentAttention" in text and "RoutedExperts" in text


def test_the_plain_model_in_portions_is_the_plain_model():
    """The oracle itself: a prompt cut in three, with borrowed latent rows, against one pass."""
    from helios_b200.weights.random_init import random_tensors
    from helios_b200.config.registry import resolve_architecture

    arch = resolve_architecture(FB_B)
    w = _f64(random_tensors(arch.build_plan(arch.parse_config(FB_B)), 1))
    toks = random_tokens(FB_B["vocab"], 23, 2)
    whole, streams, _ = pf.forward(FB_B, w, toks)
    assert streams.shape == (4, 23, 50)
    past, parts = None, []
    for a, b in [(0, 9), (9, 11), (11, 23)]:
        logits, _s, past = pf.forward(FB_B, w, toks[a:b], past)
        parts.append(logits)
    assert (torch.cat(parts) - whole).abs().max() < 1e-9


def test_the_plain_choice_of_experts():
    ro = {"top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([[4.0, 0.0, 5.0, 0.5, 4.5, 1.0]], dtype=torch.float64)
    idx, wts = pf.router_choice(z, ro)
    assert sorted(idx[0].tolist()) == [2, 3]              # expert 4 has the second score, but its group loses
    s = torch.softmax(z, -1)[0]
    assert abs(float(wts.sum()) - 3.0) < 1e-9 and abs(float(wts[0, 0]) - 3.0 * float(s[2] / (s[2] + s[3]))) < 1e-9
    idx, _ = pf.router_choice(z, {"top": 2})
    assert sorted(idx[0].tolist()) == [2, 4]
    idx, _ = pf.router_choice(z, dict(ro, groups={"count": 3, "keep": 2}))
    assert sorted(idx[0].tolist()) == [2, 4]


# ====================================================================== kernels on made inputs
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_times_a_constant(dtype):
    from helios_b200.csrc import ops

    table = torch.randn(11, 24).to(_dt(dtype))
    ids = torch.tensor([3, 0, 10, 3], dtype=torch.int32)
    got = ops.embedding(ids.cuda(), table.cuda(), 7.5).cpu()
    assert got.dtype == torch.float32 and torch.equal(got, table.float()[ids.long()] * 7.5)
    assert torch.equal(ops.embedding(ids.cuda(), table.cuda()).cpu(), table.float()[ids.long()])


@pytest.mark.gpu
@pytest.mark.parametrize("pairing", ["neighbours", "halves"])
@pytest.mark.parametrize("dtype,nh,nkv,hd,vd,rot,own_values,norm", [
    ("float32", 4, 2, 24, 24, 8, True, True), ("float32", 3, 3, 10, 14, 10, True, True),
    ("bfloat16", 4, 1, 64, 64, 16, True, True), ("bfloat16", 6, 2, 96, 96, 96, True, True),
    ("float32", 5, 1, 40, 40, 0, True, True), ("bfloat16", 2, 2, 32, 32, 2, True, True),
    ("bfloat16", 4, 2, 64, 40, 32, True, True), ("bfloat16", 3, 1, 20, 20, 6, True, True),
    ("float32", 4, 2, 16, 16, 6, False, False), ("bfloat16", 8, 4, 128, 128, 64, False, False),
    ("bfloat16", 4, 2, 32, 32, 8, False, True), ("float32", 2, 1, 12, 12, 12, False, True)])
def test_norm_over_whole_projections_neighbour_rotation_and_the_cache_write(dtype, nh, nkv, hd, vd, rot, own_values,
                                                                            norm, pairing):
    """q and k normed over all heads at once with weights of that size, THEN rotated (in
    neighbouring pairs, or value i with value i + rot / 2) on the first ``rot`` values of every head; k to the key pages, v (columns
    of its own, or the keys as projected) to the value pages; pages in a scrambled order."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(hd + rot + nh)
    page, eps, base = 8, 1e-5, 300.0
    positions = torch.tensor([0, 1, 7, 8, 9, 40, 3], dtype=torch.int32)
    seq_of = torch.tensor([0, 0, 0, 0, 0, 0, 1], dtype=torch.int32)
    T = len(positions)
    v_col = (nh + nkv) * hd if own_values else None
    ld = (nh + nkv) * hd + (nkv * vd if own_values else 0) + 8
    rows = torch.randn(T, ld, generator=g).to(dt)
    table = torch.tensor([[5, 2, 9, 0, 7, 1], [3, 4, 6, 8, 10, 11]], dtype=torch.int32)
    kp = torch.full((12, nkv, page, hd), float("nan"), dtype=dt)
    vp = torch.full((12, nkv, page, vd), float("nan"), dtype=dt)
    wq = (1.0 + 0.3 * torch.randn(nh * hd, generator=g)) if norm else None
    wk = (1.0 + 0.3 * torch.randn(nkv * hd, generator=g)) if norm else None
    rcfg = {"dims": rot, "base": base}
    cos = sin = None
    if rot:
        f, _ = pf.rotary_frequencies(rcfg)
        a = positions.double()[:, None] * f[None, :]
        cos, sin = torch.cos(a).float().cuda(), torch.sin(a).float().cuda()
    r, kpd, vpd = rows.cuda(), kp.cuda(), vp.cuda()
    ops.qk_rotate_norm_write(r, cos, sin, positions.cuda(), seq_of.cuda(), table.cuda(), kpd, vpd, nh, nkv, hd, vd,
                             page, "row" if norm else False, wq.cuda() if norm else None,
                             wk.cuda() if norm else None, eps, v_col, write_cache=True, pairing=pairing)
    rotate = pf.rotate_neighbours if pairing == "neighbours" else pf.rotate_halves
    x = rows.double()
    q, k = x[:, :nh * hd], x[:, nh * hd:(nh + nkv) * hd]
    if norm:
        q, k = pf.rms_norm(q, wq.double(), eps), pf.rms_norm(k, wk.double(), eps)
    q, k = q.reshape(T, nh, hd), k.reshape(T, nkv, hd)
    if rot:
        q, k = rotate(q, positions, rcfg), rotate(k, positions, rcfg)
    v = x[:, v_col:v_col + nkv * vd].reshape(T, nkv, vd) if own_values else x[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    got_q = r.float().cpu().double()[:, :nh * hd].reshape(T, nh, hd)
    assert (got_q - q).abs().max() < tol * max(1.0, float(q.abs().max()))
    kc, vc = kpd.float().cpu().double(), vpd.float().cpu().double()
    for t in range(T):
        pg, slot = int(table[seq_of[t], positions[t] // page]), int(positions[t]) % page
        assert (kc[pg, :, slot] - k[t]).abs().max() < tol * max(1.0, float(k.abs().max())), t
        assert torch.equal(vc[pg, :, slot], v[t]), t                    # values go as they are
    written = torch.zeros(12, page, dtype=torch.bool)
    for t in range(T):
        written[int(table[seq_of[t], positions[t] // page]), int(positions[t]) % page] = True
    assert torch.isnan(kc.transpose(1, 2)[~written]).all() and torch.isnan(vc.transpose(1, 2)[~written]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,heads,nope,rot,rank,q_rank,nrot,pairing", [
    ("float32", 2, 10, 6, 20, 7, 6, "halves"), ("bfloat16", 4, 32, 16, 64, 40, 16, "halves"),
    ("float32", 3, 8, 8, 12, 9, 4, "halves"), ("bfloat16", 4, 16, 32, 96, 128, 32, "neighbours"),
    ("float32", 1, 4, 2, 5, 3, 2, "halves")])
def test_query_latent_norm_latent_rows_and_rotation_of_halves(dtype, heads, nope, rot, rank, q_rank, nrot, pairing):
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(rank + rot)
    page, eps = 4, 1e-5
    positions = torch.tensor([0, 3, 4, 5, 21, 2], dtype=torch.int32)
    seq_of = torch.tensor([0, 0, 0, 0, 0, 1], dtype=torch.int32)
    T = len(positions)
    table = torch.tensor([[5, 2, 9, 0, 7, 1], [3, 4, 6, 8, 10, 11]], dtype=torch.int32)
    first = torch.randn(T, q_rank + rank + rot + 3, generator=g).to(dt)         # [query latent | latent | key part | more]
    q = torch.randn(T, heads * (nope + rot), generator=g).to(dt)
    wn, wqn = 1 + 0.3 * torch.randn(rank, generator=g), 1 + 0.3 * torch.randn(q_rank, generator=g)
    rcfg = {"dims": nrot, "base": 50.0}
    f, _ = pf.rotary_frequencies(rcfg)
    a = positions.double()[:, None] * f[None, :]
    cos, sin = torch.cos(a).float().cuda(), torch.sin(a).float().cuda()
    pages = torch.full((12, 1, page, rank + rot), float("nan"), dtype=dt).cuda()
    fd, qd = first.cuda(), q.cuda()
    args = (cos, sin, positions.cuda(), seq_of.cuda(), table.cuda(), heads, nope, rot, rank, page, eps)
    apart = torch.full((T, q_rank), float("nan"), dtype=dt).cuda()        # the normed query latent in rows of its own
    ops.latent_prepare_parts(None, None, fd[:, :q_rank], None, None, wqn.cuda(), *args, pairing=pairing,
                             query_latent_out=apart)
    assert torch.equal(fd.cpu(), first)
    ops.latent_prepare_parts(None, fd[:, q_rank:q_rank + rank + rot], fd[:, :q_rank], pages, wn.cuda(), wqn.cuda(),
                             *args, write_cache=True, pairing=pairing)
    assert torch.equal(apart, fd[:, :q_rank])
    ops.latent_prepare_parts(qd, None, None, None, None, None, *args, pairing=pairing)
    rotate = pf.rotate_halves if pairing == "halves" else pf.rotate_neighbours
    x = first.double()
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    want_cq = pf.rms_norm(x[:, :q_rank], wqn.double(), eps)
    assert (fd.float().cpu().double()[:, :q_rank] - want_cq).abs().max() < tol * float(want_cq.abs().max())
    assert torch.equal(fd.cpu()[:, q_rank:], first[:, q_rank:])                  # the rest of the rows stays
    want_c = pf.rms_norm(x[:, q_rank:q_rank + rank], wn.double(), eps)
    want_kr = rotate(x[:, q_rank + rank:q_rank + rank + rot], positions, rcfg)
    pc = pages.float().cpu().double()
    for t in range(T):
        pg, slot = int(table[seq_of[t], positions[t] // page]), int(positions[t]) % page
        assert (pc[pg, 0, slot, :rank] - want_c[t]).abs().max() < tol * float(want_c.abs().max())
        assert (pc[pg, 0, slot, rank:] - want_kr[t]).abs().max() < tol * float(want_kr.abs().max())
    qq = q.double().reshape(T, heads, nope + rot)
    want_q = torch.cat([qq[..., :nope], rotate(qq[..., nope:], positions, rcfg)], -1)
    assert (qd.float().cpu().double().reshape(T, heads, -1) - want_q).abs().max() < tol * float(want_q.abs().max())
    # a layer that reads another layer's rows: nothing is written
    before = pages.clone()
    ops.latent_prepare_parts(None, None, fd[:, :q_rank], pages, None, wqn.cuda(), *args, write_cache=False,
                             pairing=pairing)
    assert torch.equal(torch.nan_to_num(before.float()), torch.nan_to_num(pages.float()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,T,H,N", [("float32", 5, 3, 6), ("bfloat16", 40, 4, 32), ("bfloat16", 3, 2, 12),
                                         ("float32", 70, 6, 16)])
def test_gate_on_every_value_of_heads_that_lie_apart(dtype, T, H, N):
    """The heads' outputs as a batched product leaves them (head-major) and as rows; the gate a
    column slice of wider rows."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(H, T, N, generator=g).to(dt)
    wide = (3 * torch.randn(T, H * N + 16, generator=g)).to(dt)
    want = x.double().transpose(0, 1).reshape(T, H * N) * torch.sigmoid(wide.double()[:, 8:8 + H * N])
    tol = 1e-6 if dtype == "float32" else 1e-2
    for view in (x.cuda().transpose(0, 1), x.transpose(0, 1).contiguous().cuda()):
        got = ops.gate_heads(view, wide.cuda()[:, 8:8 + H * N])
        assert got.is_contiguous() and (got.float().cpu().double() - want).abs().max() < tol * float(want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("experts,top,groups,scale", [(12, 4, (3, 2), 1.5), (8, 2, (4, 2), 1.0), (6, 3, None, 2.0),
                                                      (6, 1, (3, 1), 1.0), (6, 2, (6, 6), 0.5), (7, 7, (1, 1), 1.0),
                                                      (64, 8, (8, 3), 2.5), (256, 6, (32, 4), 1.0), (40, 3, (20, 2), 1.0)])
def test_choice_among_the_best_groups_with_normalised_scaled_weights(experts, top, groups, scale):
    from helios_b200.csrc import ops

    g = torch.Generator().manual_seed(experts + top)
    z = torch.randn(300, experts, generator=g) * 2.0
    ro = {"top": top, "scale": scale}
    if groups:
        ro["groups"] = {"count": groups[0], "keep": groups[1]}
    want_ids, want_w = pf.router_choice(z.double(), ro)
    plain_ids, _ = pf.router_choice(z.double(), {"top": top})
    ids, wts = ops.moe_topk(z.cuda(), top, "softmax", groups=groups, normalize=True, scale=scale)
    ids, wts = ids.cpu().long(), wts.cpu().double()
    assert torch.equal(ids.sort(-1).values, want_ids.sort(-1).values)
    if groups and groups[1] < groups[0] and top > groups[1]:
        assert not torch.equal(want_ids.sort(-1).values, plain_ids.sort(-1).values)      # the limit shows
    order = want_ids.argsort(-1)
    assert (wts.gather(1, ids.argsort(-1)) - want_w.gather(1, order)).abs().max() < 1e-5 * scale
    assert (wts.sum(-1) - scale).abs().max() < 1e-5 * scale
    # a row of NaN (the padding of a captured step) still yields distinct eligible ids
    ids, _ = ops.moe_topk(torch.full((3, experts), float("nan")).cuda(), top, "softmax", groups=groups,
                          normalize=True, scale=scale)
    assert all(len(set(r.tolist())) == top and min(r.tolist()) >= 0 and max(r.tolist()) < experts for r in ids.cpu())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,top,groups", [(64, 24, 9, 2, (3, 2)), (50, 12, 6, 3, None), (128, 48, 4, 4, (2, 2))])
def test_routed_feed_forward_alone(dtype, width, ff, experts, top, groups):
    from helios_b200.parts import part_class

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(width + ff)
    part = part_class("feed_forward", "routed_experts")(width, ff, experts, top, 1.5, router="softmax",
                                                        weight_on="output", activation="clamped_swish",
                                                        groups=groups, normalize=True, weight_scale=1.25)
    t = {}
    for name, spec in part.weight_specs().items():
        t[name] = (torch.randn(spec.shape, generator=g) * 0.3).to(dt).float()
    h = torch.randn(80, width, generator=g).to(dt).float()
    ro = {"top": top, "scale": 1.25}
    if groups:
        ro["groups"] = {"count": groups[0], "keep": groups[1]}
    z = h.double() @ t["router"].double().T
    # tokens whose choice rounding cannot change: every two logits (so every two scores, and
    # every two groups' bests) well apart
    srt = z.sort(-1).values
    h = h[(srt[:, 1:] - srt[:, :-1]).min(-1).values > 0.04]
    assert h.shape[0] > 8
    part.bind({k: v.to(dt).cuda() for k, v in t.items()})
    got = part.forward(SimpleNamespace(), h.to(dt).cuda()).float().cpu().double()
    w = {"p." + k: v.double() for k, v in t.items()}
    want = pf.routed_ff(h.double(), w, "p.", {"router": ro, "expert": {"limit": 1.5}})
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))


# ====================================================================== one key that takes all the weight
def _needle_model(kind, dtype_seed=0):
    """A one-layer model (two where a layer borrows rows) in which channel ``c0`` of the
    stream carries a mark that only the tokens A (a key) and B (a query) have: the projections
    read it into one unrotated value of every head's query and key, so that B's score against A
    stands far above every other score, wherever A sits."""
    if kind == "attention":
        layers = [(_att(4, 2, 32, 32, 1.0, _rot(8, 1000.0)), None)]
    elif kind == "attention_2":
        layers = [(_att2(4, 2, 32, 1.0, _rot(8, 1000.0)), None)]
    else:
        layers = [(_lat(4, 32, 16, 32, 32, 24, 1.0, 1000.0), None)]
        if kind == "latent_borrowed":
            layers.append((_lat(2, 16, 16, 24, 32, 16, 1.0, 1000.0, kv_from=0), None))
    return _model(61, 64, 1e-5, 2.0, layers)


def _needle_weights(cfg, weights, A=7, B=9, c0=5, c1=6, mark=3.0, gain=6.0):
    """Token A alone carries a mark in channel c0, which only the key projections read, token B
    alone one in channel c1, which only the query projections read."""
    w = {k: v.clone() for k, v in weights.items()}
    w["embed"][:, c0] = w["embed"][:, c1] = 0.0
    w["embed"][A, c0] = w["embed"][B, c1] = mark
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.mix.", layer["mixer"]
        w[p + "o"] *= 40.0                            # what the query attends decides the logits
        w[p + "o"][[c0, c1], :] = 0.0                 # the marks stay as the embedding left them
        w[f"l{i}.norm1"][[c0, c1]] = 1.0
        d = mx["dim"]
        if layer["type"] in ("attention", "attention_2"):
            col = d - 1                               # a value of the head that is not rotated
            for h in range(mx["heads"]):
                w[p + "q"][h * d + col, :] = 0.0
                w[p + "q"][h * d + col, c1] = gain
            for h in range(mx["kv_heads"]):
                w[p + "k"][h * d + col, :] = 0.0
                w[p + "k"][h * d + col, c0] = gain
            if layer["type"] == "attention":
                w[p + "q.norm"][:] = 3.0
                w[p + "k.norm"][:] = 3.0
        else:
            step = d + mx["rot_dim"]
            w[p + "dq"][0, :] = 0.0
            w[p + "dq"][0, c1] = gain                 # the query latent's value 0 carries B's mark ...
            w[p + "uq"][:, 0] = 0.0
            w[p + "uk"][:, 0] = 0.0
            for h in range(mx["heads"]):              # ... into unrotated value 0 of every head's query
                w[p + "uq"][h * step, :] = 0.0
                w[p + "uq"][h * step, 0] = gain
                w[p + "uk"][h * d, :] = 0.0           # and the latent's value 0 into that value of the key
                w[p + "uk"][h * d, 0] = gain
            if "kv_from" not in mx:
                w[p + "dkv"][0, :] = 0.0
                w[p + "dkv"][0, c0] = gain            # the latent's value 0 carries A's mark
    return w


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "attention_2", "latent", "latent_borrowed"])
def test_one_key_that_takes_all_the_weight_wherever_it_sits(kind, dtype, tmp_path):
    """The marked key at position 0, at a page's last place, at the next page's first, just
    before the query, and hundreds of tokens back; the marked query in a prompt, in a later
    portion, and decoded alone.  The plain model says the query's weight is on that key."""
    from safetensors.torch import save_file
    from helios_b200.engine.batch import StepEntry
    from helios_b200.weights import write_model_folder

    cfg = _needle_model(kind)
    folder = write_model_folder(tmp_path / kind, cfg, 11)
    _c, weights = read_folder(folder)
    weights = _needle_weights(cfg, weights)
    save_file(weights, str(folder / "model.safetensors"))
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    A, B, n = 7, 9, 420
    filler = [t for t in random_tokens(cfg["vocab"], 2 * n, 5) if t not in (A, B)][:n]
    core = _core(folder, dtype, 1024)
    # the mark does take the weight: without the key the query's output is another one
    probe = list(filler[:40])
    probe[3], probe[39] = A, B
    with_key = pf.forward(cfg, w, probe)[0][39]
    probe[3] = filler[3]
    assert (with_key - pf.forward(cfg, w, probe)[0][39]).abs().max() > 0.05 * float(with_key.abs().max())
    for case, where in enumerate([0, 15, 16, 17, 31, 32, 200, 418]):
        toks = list(filler)
        toks[where], toks[n - 1] = A, B
        want = pf.forward(cfg, w, toks)[0]
        rid = f"{kind}{case}"
        cuts = {0: [n], 1: [n - 1, 1], 2: [where + 1, n - where - 2, 1] if where < n - 2 else [n - 1, 1],
                3: [16, 16, n - 33, 1]}[case % 4]
        at, rows = 0, []
        for c in cuts:
            if c <= 0:
                continue
            out = core.step([StepEntry(rid, toks[at:at + c], [c - 1])])
            rows.append((at + c - 1, out))
            at += c
        core.end(rid)
        pos, got = rows[-1]
        assert pos == n - 1
        from conftest import assert_logits_close
        assert_logits_close(got, want[pos:pos + 1], dtype, f"{kind}: key at {where}, cuts {cuts}")


# ====================================================================== whole models
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FB_ALONE) + list(FB_CONFIGS))
def test_whole_prompts_and_the_stream_after_every_layer(fb_folders, name, dtype):
    """Logits at every position of whole prompts (the first tokens of a sequence among them),
    and the residual stream after every layer."""
    cfg, weights = read_folder(fb_folders[name])
    reqs = _requests(cfg, [1, 2, 3, 41, 130], 100)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.whole(tb, rid, toks)
    core = _core(fb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} whole")
    from helios_b200.engine.batch import StepEntry
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    _, want_layers, _ = pf.forward(cfg, w, reqs["q3"])
    seen = []

    def recording(inner):
        def forward(*args):
            residual, pending = inner(*args)
            x = residual.detach().double().cpu().clone()
            for t, _s in pending.terms:
                x += t.double().cpu()
            seen.append(x)
            return residual, pending
        return forward

    for blk in core.model.plan.layers:
        blk.forward = recording(blk.forward)
    core.step([StepEntry("layers", reqs["q3"], [0])])
    assert len(seen) == want_layers.shape[0]
    for i, (got, want) in enumerate(zip(seen, want_layers)):
        tol = 2e-5 * max(1.0, float(want.abs().max())) if dtype == "float32" else 3e-2 * float(want.abs().max())
        assert (got - want).abs().max() < tol, f"{name}: residual after layer {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FB_CONFIGS))
def test_prefill_then_long_decoding_token_by_token(fb_folders, name, dtype):
    """Most of the prompt in one step, then 70 single tokens (captured decode steps) that pass
    page borders, up to position 260."""
    cfg, weights = read_folder(fb_folders[name])
    reqs = _requests(cfg, [75, 131, 260], 200)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.prefill_then_decode(tb, rid, toks, n_decode=70)
    core = _core(fb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} decode")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FB_CONFIGS))
def test_portions_of_changing_size_down_to_one_token(fb_folders, name, dtype):
    cfg, weights = read_folder(fb_folders[name])
    reqs = _requests(cfg, [64, 97, 50, 33], 300)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    sizes = [[7], [2, 31, 3, 16, 2, 17], [1, 2, 1, 1, 3, 13, 2, 1, 5], [16, 1, 15, 1]]
    for (rid, toks), sz in zip(reqs.items(), sizes):
        tu.portions(tb, rid, toks, sz)
    core = _core(fb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} portions")


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FB_CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(fb_folders, name, dtype, graphs):
    """Nine unequal requests through three slots: portions of some beside single tokens of
    others; every finished request's pages and slot go to the next."""
    cfg, weights = read_folder(fb_folders[name])
    reqs = _requests(cfg, [40, 23, 77, 18, 52, 31, 66, 20, 45], 400)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=7, max_live=3, decode_tail=10)
    core = _core(fb_folders[name], dtype, tb.live_tokens_peak, max_slots=3, graphs=graphs)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} mixed")
    assert core.cache.num_free_slots == 3 and all(p.num_used == 0 for p in core.cache.pools)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["fb_a", "fb_b"])
def test_a_batch_gives_each_request_what_it_gets_alone(fb_folders, name):
    """float32: the same rows bit for bit, alone or beside others, in one step or in portions,
    whatever the slots and pages."""
    from helios_b200.engine.batch import StepEntry

    cfg, _w = read_folder(fb_folders[name])
    reqs = _requests(cfg, [37, 5, 60], 500)
    core = _core(fb_folders[name], "float32", 512, max_slots=4)
    alone = {}
    for rid, toks in reqs.items():
        alone[rid] = core.step([StepEntry(rid, toks, range(len(toks)))]).clone()
        core.end(rid)
    core.step([StepEntry("other", random_tokens(cfg["vocab"], 21, 1), [0])])      # shifts slots and pages
    got = core.step([StepEntry(rid, toks, range(len(toks))) for rid, toks in reqs.items()])
    off = 0
    for rid, toks in reqs.items():
        assert torch.equal(got[off:off + len(toks)], alone[rid]), rid
        off += len(toks)
    for rid in reqs:
        core.end(rid)
    toks = reqs["q2"]
    parts = [core.step([StepEntry("cut", toks[a:b], range(b - a))]) for a, b in [(0, 2), (2, 31), (31, 33), (33, 60)]]
    assert torch.equal(torch.cat(parts), alone["q2"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_through_trace_run(fb_folders, dtype, tmp_path):
    cfg, weights = read_folder(fb_folders["fb_b"])
    reqs = _requests(cfg, [30, 47, 22, 39, 28], 600)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=3, max_live=4, decode_tail=8)
    got = tu.run_trace_run(fb_folders["fb_b"], dtype, tb, tmp_path / "out", tb.live_tokens_peak, cfg["vocab"])
    tu.check(tb, got, plain, dtype, "fb_b trace_run")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["fb_a", "fb_b"])
def test_greedy_generation_through_the_scheduler(fb_folders, name, dtype):
    from helios_b200 import LLM, SamplingParams

    cfg, weights = read_folder(fb_folders[name])
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 5, 17, 33, 9, 26)]
    llm = LLM(str(fb_folders[name]), dtype=dtype, kv_cache_bytes=1 << 22, max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(max_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 12
        toks = list(prompt)
        for t in out.token_ids:
            logits = pf.forward(cfg, w, toks)[0][-1]
            best = int(torch.argmax(logits))
            if t != best:
                assert dtype == "bfloat16", f"token {t} instead of {best} after {len(toks)} tokens"
                assert float(logits[best] - logits[t]) <= 0.03 * float(logits.abs().max())
            toks.append(t)
