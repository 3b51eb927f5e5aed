"""The Gebasun design against a plain float64 implementation (``plain_gebasun``): every
mechanism alone on made inputs, then whole models of several shapes through the step function
(whole prompts, decoding, portions, mixed batches, replay, generation)."""
from __future__ import annotations

import json
import math
from types import SimpleNamespace

import pytest
import torch

import plain_gebasun as pg
import trace_util as tu
from conftest import random_tokens, read_folder

DTYPES = ["float32", "bfloat16"]


# ---------------------------------------------------------------------- configurations
def _att(heads, kv, dim, scale, size, rows, far):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                                           "bias_max": far, "bias_rows": rows, "mask": {"size": size}}}


def _att2(heads, kv, dim, scale, size, keep, rot, base):
    mask = {"size": size}
    if keep is not None:
        mask["keep_first"] = keep
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                                             "mask": mask, "rot": {"dims": rot, "base": base}}}


def _ssm(heads, vdim, state, groups, conv, parts):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "conv": conv, "norm_groups": parts}}


def _moe(ff, experts, top, shared=None):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


def _model(vocab, width, eps, layers):
    return {"architecture": "Gebasun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


# heads of 32 (the tensor-core kernels' smallest), windows shorter than the prompts, every mixer
GB_A = _model(211, 96, 1e-5, [
    (_att(4, 2, 32, 0.2, 24, 12, 40), _moe(40, 6, 2, 32)),
    (_att2(4, 1, 32, 0.18, 20, 5, 16, 10000.0), _moe(40, 6, 2, 32)),
    (_ssm(4, 24, 16, 2, 4, 2), _moe(40, 6, 2, 32)),
    (_ssm(4, 24, 16, 2, 4, 2), None),
])
# another order, one head a group, a full rotation, no kept tokens, an odd bias table, a
# window longer than most prompts, one expert a token, no shared expert, three taps
GB_B = _model(150, 80, 3e-6, [
    (_ssm(5, 16, 24, 5, 3, 1), _moe(24, 3, 1)),
    (_att2(5, 5, 24, 0.25, 33, None, 24, 500.0), None),
    (_att(6, 3, 40, 0.15, 100, 9, 50), _moe(20, 3, 1)),
])
# heads of 64, more kept tokens than a page, all experts chosen, one group, two taps
GB_C = _model(180, 128, 1e-5, [
    (_att2(8, 2, 64, 0.125, 44, 19, 32, 300000.0), _moe(48, 4, 4, 16)),
    (_att(8, 4, 64, 0.11, 30, 32, 110), _moe(48, 4, 4, 16)),
    (_ssm(8, 32, 64, 1, 2, 4), _moe(48, 4, 4, 16)),
])
# a width that is no multiple of 8, heads of 10, a window of one page, a single tap
GB_D = _model(131, 50, 2e-6, [
    (_att(5, 1, 10, 0.4, 16, 6, 12), _moe(12, 5, 3, 9)),
    (_ssm(2, 15, 7, 1, 1, 3), _moe(12, 5, 3, 9)),
    (_att2(2, 2, 10, 0.3, 17, 16, 2, 77.0), _moe(12, 5, 3, 9)),
])
GB_CONFIGS = {"gb_a": GB_A, "gb_b": GB_B, "gb_c": GB_C, "gb_d": GB_D}
GB_SEEDS = {"gb_a": 3, "gb_b": 4, "gb_c": 5, "gb_d": 6}
GB_ALONE = {
    "bias_attention_only": _model(97, 64, 1e-5, [(_att(4, 2, 16, 0.3, 21, 8, 30), None)]),
    "rotary_attention_only": _model(97, 64, 1e-5, [(_att2(4, 2, 16, 0.3, 19, 3, 8, 1000.0), None)]),
    "state_space_only": _model(97, 64, 1e-5, [(_ssm(4, 8, 12, 2, 4, 2), None)]),
    "routed_ff": _model(97, 64, 1e-5, [(_ssm(2, 8, 8, 1, 2, 1), _moe(24, 6, 2, 32))]),
}


def _wide_router_margins(cfg, weights):
    """Make every routed layer's choice a matter of the token id with margins far beyond
    rounding, so that bfloat16 and float64 choose alike.  Channels 0..E-1 of the embedding hold a
    code (the token's j-th choice gets 4 - j); no output projection writes to those channels,
    so the stream keeps the code; the feed-forward's norm passes them with weight 1 (a common
    positive factor 1 / rms keeps their order); router row e reads the channels c with
    c % experts == e; the router's bias stays small beside the code's steps."""
    w = {k: v.clone() for k, v in weights.items()}
    routed = [l["mlp"] for l in cfg["layers"] if l.get("mlp")]
    if not routed:
        return w
    E = max(ml["router"]["experts"] for ml in routed)
    assert cfg["width"] > E
    w["embed"][:, :E] = 0.0
    for i, layer in enumerate(cfg["layers"]):
        w[f"l{i}.mix.o"][:E, :] = 0.0
        if f"l{i}.mix.o.b" in w:
            w[f"l{i}.mix.o.b"][:E] = 0.0
        ml = layer.get("mlp")
        if not ml:
            continue
        n_out = ml["router"]["experts"]
        for name in [f"l{i}.mlp.e{e}.down" for e in range(n_out)] + [f"l{i}.mlp.shared.down"]:
            if name in w:
                w[name][:E, :] = 0.0
        w[f"l{i}.norm2"][:E] = 1.0
        r = w[f"l{i}.mlp.router"]
        r[:, :] = 0.0
        for c in range(E):
            r[c % n_out, c] = 1.0
        w[f"l{i}.mlp.router.b"] = 0.1 * torch.randn(n_out, generator=torch.Generator().manual_seed(i))
    w["final.norm"][:E] = 0.05
    top_most = max(ml["router"]["top"] for ml in routed)
    for tok in range(cfg["vocab"]):
        for j in range(min(top_most, E)):
            w["embed"][tok, (tok + j) % E] = 4.0 - 0.8 * j
    return w


@pytest.fixture(scope="module")
def gb_folders(tmp_path_factory):
    """Model folders with random weights; ``config.json`` is then written WITHOUT the rows of
    the distance-bias tables, which a reader has to take from the tensors' shapes."""
    from safetensors.torch import save_file
    from helios_b200.weights import write_model_folder

    out = {}
    base = tmp_path_factory.mktemp("gebasun")
    for name, cfg in {**GB_CONFIGS, **GB_ALONE}.items():
        folder = write_model_folder(base / name, cfg, GB_SEEDS.get(name, 9))
        _cfg, weights = read_folder(folder)
        save_file(_wide_router_margins(cfg, weights), str(folder / "model.safetensors"))
        lean = json.loads(json.dumps(cfg))
        for layer in lean["layers"]:
            layer["mixer"].pop("bias_rows", None)
        (folder / "config.json").write_text(json.dumps(lean))
        out[name] = folder
    return out


def _bf16(weights):
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 and not k.endswith((".rel", ".conv")) else v.float())
            for k, v in weights.items()}


def _f64(weights):
    return {k: v.double() for k, v in weights.items()}


def _plain(cfg, weights, dtype, requests):
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    return {rid: pg.model(cfg, w, toks)[0] for rid, toks in requests.items()}


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
    from helios_b200.config.gebasun_config import (BiasAttentionConfig, GebasunConfig, RotaryAttentionConfig,
                                                   StateSpaceConfig)

    cfg = GebasunConfig.from_json(GB_B)
    assert [type(l.mixer) for l in cfg.layers] == [StateSpaceConfig, RotaryAttentionConfig, BiasAttentionConfig]
    assert cfg.layers[1].mixer.keep_first == 0 and cfg.layers[1].mlp is None
    assert cfg.layers[2].mixer.bias_rows == 9 and cfg.layers[2].mixer.bias_max == 50.0
    assert cfg.layers[0].mlp.shared_ff is None and cfg.layers[0].mlp.top == 1
    assert GebasunConfig.from_json(GB_C).layers[0].mixer.keep_first == 19
    for path, value, word in [(("layers", 0, "mixer", "state"), None, "state"),
                              (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
                              (("layers", 2, "mixer", "vdim"), 8, "vdim"),
                              (("layers", 2, "mlp", "router", "top"), 9, "top"),
                              (("layers", 0, "type"), "conv", "type"),
                              (("norm",), {}, "eps")]:
        bad = json.loads(json.dumps(GB_B))
        at = bad
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            GebasunConfig.from_json(bad)


def test_plan_names_every_tensor_and_sizes_caches_and_state():
    from helios_b200.cache.manager import cache_groups_of
    from helios_b200.config.gebasun_config import GebasunConfig
    from helios_b200.models import build_gebasun_plan
    from helios_b200.weights.loader import expected_tensors

    plan = build_gebasun_plan(GebasunConfig.from_json(GB_A))
    names = expected_tensors(plan)
    for name in ["embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.b",
                 "l0.mix.rel", "l0.mix.sink", "l0.mix.o.b", "l1.mix.g", "l1.mix.sink", "l2.mix.in", "l2.mix.conv",
                 "l2.mix.conv.b", "l2.mix.dt_bias", "l2.mix.A_log", "l2.mix.D", "l2.mix.norm", "l2.mix.o",
                 "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e5.up", "l0.mlp.e5.down", "l0.mlp.shared.up", "l3.norm1"]:
        assert name in names, name
    for name in ["l0.mix.v", "l0.mix.g", "l1.mix.rel", "l1.mix.o.b", "l0.mlp.e0.gate", "l3.norm2", "l3.mlp.router"]:
        assert name not in names, name
    assert names["l2.mix.in"][2].shape == (2 * 96 + 2 * 2 * 16 + 4, 96)
    assert names["l1.mix.g"][2].shape == (4 * 32, 96) and names["l0.mix.rel"][2].shape == (12, 4)
    specs, where = cache_groups_of(plan)
    assert sorted(where) == [0, 1]
    by_window = {s.window: s for s in specs}
    assert by_window[24].keep_first == 0 and by_window[20].keep_first == 5 and by_window[20].num_kv_heads == 1
    ssm = plan.layers[2].mixer
    assert ssm.state_spec().shape == (4 * 16 * 24 + (96 + 64) * 3,)


def test_toy_model_of_the_design_from_the_command_line(tmp_path, capsys):
    from helios_b200 import cli

    assert cli.main(["make-toy-model", "--arch", "gebasun", "--out", str(tmp_path / "toy"), "--layers", "4",
                     "--hidden", "64", "--heads", "4", "--kv-heads", "2"]) == 0
    assert cli.main(["info", "--model", str(tmp_path / "toy")]) == 0
    text = capsys.readouterr().out
    assert "Gebasun" in text and "SelectiveStateMixer" in text and "RoutedExperts" in text


def test_buckets_of_the_distance_bias():
    from helios_b200.csrc.ops import distance_bias_rows

    for rows, far in [(12, 40.0), (9, 50.0), (32, 120.0), (6, 12.0), (16, 64.0), (64, 512.0)]:
        b = [pg.distance_bucket(n, rows, far) for n in range(int(far) + 40)]
        assert b[:rows // 2] == list(range(rows // 2)) and b[rows // 2] == rows // 2
        assert all(x <= y for x, y in zip(b, b[1:])) and max(b) == rows - 1
        assert all(x == rows - 1 for x in b[int(math.ceil(far)):])
        table = torch.randn(rows, 3)
        flat = distance_bias_rows(table, far)
        assert flat.shape[0] <= int(far) + 3
        for n in range(int(far) + 40):
            assert torch.equal(flat[min(n, flat.shape[0] - 1)], table[b[n]]), (rows, far, n)
        short = distance_bias_rows(table, far, window=7)
        assert short.shape[0] == min(7, flat.shape[0]) and torch.equal(short, flat[:short.shape[0]])


def test_pages_behind_a_window_go_back_but_the_first_tokens_stay():
    from helios_b200.cache.pages import CacheLayout, GroupLayout

    lay = CacheLayout([GroupLayout(20, 12, keep_first=17), GroupLayout(None, 12), GroupLayout(24, 12)], 8, 2)
    lay.admit("a")
    for n in [5, 30, 1, 1, 40, 3]:
        lay.extend("a", n)
        lay.commit("a", n)
        lay.check_invariants()
    L = lay.length("a")
    assert L == 80
    t0, t1, t2 = (lay.table("a", g) for g in range(3))
    first_needed = (L - 20 + 1) // 8
    assert all(p >= 0 for p in t0[:3]) and all(p < 0 for p in t0[3:first_needed]) and all(p >= 0 for p in t0[first_needed:])
    assert all(p >= 0 for p in t1)
    assert all(p < 0 for p in t2[:(L - 24 + 1) // 8])
    assert lay.pages_held("a")[0] == 3 + len(t0) - first_needed
    assert lay.peak_pages(0, 1000, 16) == -(-(20 + 16) // 8) + 1 + 3
    lay.admit("b")
    lay.extend("b", 9)
    lay.commit("b", 9)           # takes pages "a" gave back
    lay.check_invariants()
    lay.release("a")
    lay.release("b")
    lay.check_invariants()
    assert all(p.num_used == 0 for p in lay.pools)


# ====================================================================== kernels on made inputs
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [50, 96, 1024])
def test_two_norms_of_one_row_with_the_pending_add(dtype, width):
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(width)
    res = torch.randn(7, width, generator=g)
    a = torch.randn(7, width, generator=g).to(dt)
    b = torch.randn(7, width, generator=g).to(dt)
    w1, w2 = torch.randn(width, generator=g), torch.randn(width, generator=g)
    for use_a, use_b, second in [(True, True, True), (True, False, True), (False, False, True), (True, True, False)]:
        r = res.clone().cuda()
        o1, o2 = ops.add_rmsnorm_pair(r, a.cuda() if use_a else None, b.cuda() if use_b else None, w1.cuda(),
                                      w2.cuda() if second else None, 1e-5, dt)
        want = res.double() + (a.double() if use_a else 0) + (b.double() if use_b else 0)
        assert (r.cpu().double() - want).abs().max() < 1e-6
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert (o1.float().cpu().double() - pg.rms_norm(want, w1.double(), 1e-5)).abs().max() < tol * 4
        if second:
            assert (o2.float().cpu().double() - pg.rms_norm(want, w2.double(), 1e-5)).abs().max() < tol * 4
        else:
            assert o2 is None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,hd,rot", [("float32", 24, 8), ("float32", 10, 10), ("bfloat16", 64, 32),
                                          ("bfloat16", 96, 24), ("float32", 40, 0), ("bfloat16", 32, 2)])
def test_rotation_unit_norm_and_the_cache_write_with_values_from_the_keys(dtype, hd, rot):
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(hd + rot)
    nh, nkv, page, eps, base = 4, 2, 8, 1e-5, 300.0
    positions = torch.tensor([0, 1, 7, 8, 9, 40, 3], dtype=torch.int32)
    seq_of = torch.tensor([0, 0, 0, 0, 0, 0, 1], dtype=torch.int32)
    T = len(positions)
    ld = (nh + nkv) * hd + 8
    rows = torch.randn(T, ld, generator=g).to(dt)
    table = torch.tensor([[5, 2, 9, 0, 7, 1], [3, 4, 6, 8, 10, 11]], dtype=torch.int32)
    kp = torch.full((12, nkv, page, hd), float("nan"), dtype=dt)
    vp = torch.full((12, nkv, page, hd), float("nan"), dtype=dt)
    cos = sin = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        ang = positions.double()[:, None] * base ** (-2.0 * i / rot)
        cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    d_rows, d_kp, d_vp = rows.cuda(), kp.cuda(), vp.cuda()
    ops.qk_rotate_norm_write(d_rows, cos, sin, positions.cuda(), seq_of.cuda(), table.cuda(), d_kp, d_vp, nh, nkv,
                             hd, hd, page, True, None, None, eps, None)
    q = rows[:, :nh * hd].double().view(T, nh, hd)
    k = rows[:, nh * hd:(nh + nkv) * hd].double().view(T, nkv, hd)
    want_q = pg.rms_unit(pg.rotate_half(q, positions, rot, base) if rot else q, eps)
    want_k = pg.rms_unit(pg.rotate_half(k, positions, rot, base) if rot else k, eps)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert (d_rows.cpu()[:, :nh * hd].double().view(T, nh, hd) - want_q).abs().max() < tol
    assert torch.equal(d_rows.cpu()[:, nh * hd:], rows[:, nh * hd:])          # k and the rest stay as projected
    written = torch.zeros(12, page, dtype=torch.bool)
    for t in range(T):
        p = int(table[seq_of[t], positions[t] // page])
        s = int(positions[t]) % page
        written[p, s] = True
        assert (d_kp.cpu()[p, :, s].double() - want_k[t]).abs().max() < tol
        assert torch.equal(d_vp.cpu()[p, :, s], rows[t, nh * hd:(nh + nkv) * hd].view(nkv, hd))
    assert torch.isnan(d_kp.float().cpu()[:, 0][~written]).all() and torch.isnan(d_vp.float().cpu()[:, 0][~written]).all()


def _paged(keys, values, page, g, dt):
    """Scatter [n, kvh, d] rows into pages handed out in a scrambled order, NaN elsewhere."""
    n = keys.shape[0]
    n_pages = -(-n // page)
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    kp = torch.full((n_pages + 4, keys.shape[1], page, keys.shape[2]), float("nan"), dtype=dt)
    vp = torch.full((n_pages + 4, values.shape[1], page, values.shape[2]), float("nan"), dtype=dt)
    for j in range(n):
        kp[order[j // page], :, j % page] = keys[j].to(dt)
        vp[order[j // page], :, j % page] = values[j].to(dt)
    return kp, vp, order.to(torch.int32)


def _attend(ops, q, kp, vp, order, q_pos, nh, nkv, hd, page, scale, window, options, decode, n_keys,
            splits=None):
    """The queries as single decoded tokens of requests of their own (``decode``), or as ONE
    portion of consecutive tokens of one request; all read the same pages."""
    from helios_b200.engine.batch import SeqSlice

    n = q.shape[0]
    dev = "cuda"
    if decode:
        seq_of, cu = torch.arange(n, dtype=torch.int32), torch.arange(n + 1, dtype=torch.int32)
        start, seqs = q_pos.clone(), [SeqSlice(None, 0, int(p), 1, i) for i, p in enumerate(q_pos.tolist())]
    else:
        assert q_pos.tolist() == list(range(int(q_pos[0]), int(q_pos[0]) + n))
        seq_of, cu = torch.zeros(n, dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32)
        start, seqs = q_pos[:1].clone(), [SeqSlice(None, 0, int(q_pos[0]), n, 0)]
    ctx = SimpleNamespace(seq_of_token=seq_of.to(dev), positions=q_pos.to(dev), start_pos=start.to(dev),
                          context_len=(q_pos + 1).to(dev) if decode else (q_pos[-1:] + 1).to(dev),
                          extras={"decode_splits": splits} if splits else {},
                          max_context_len=n_keys, cu_tokens=cu.to(dev), decode_only=decode,
                          max_tokens_per_seq=1 if decode else n, num_tokens=n, seqs=seqs, num_seqs=len(seqs))
    table = order.view(1, -1).repeat(len(seqs), 1).contiguous().to(dev)
    return ops.attention(ctx, q.to(dev), kp.to(dev), vp.to(dev), table, nh, nkv, hd, page, window, scale,
                         options=options).float().cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("decode", [True, False, "early"])
@pytest.mark.parametrize("dtype,hd,page", [("float32", 40, 16), ("bfloat16", 64, 16), ("bfloat16", 32, 16),
                                           ("bfloat16", 96, 16), ("bfloat16", 48, 16), ("bfloat16", 128, 24),
                                           ("bfloat16", 64, 8), ("bfloat16", 96, 32), ("bfloat16", 128, 16),
                                           ("bfloat16", 128, 32)])
def test_attention_singles_out_keys_at_every_edge(dtype, hd, page, decode):
    """One request of 300 tokens in scrambled pages of 16 (or 8, 24, 32), a window of 37 and 21 kept first
    tokens, a bias table, learned sinks and a gate per value.  Every query is aligned with ONE
    key and scaled so that this key, if it is visible, takes nearly all the weight whatever its
    bias: the oldest key inside the window and the one just outside, the last kept token and
    the first that is not, keys at page borders, position 0, the query's own.  A key that is
    NOT visible must leave no trace.  Then queries against which every key scores far below
    the sink.  Every row also against the plain softmax.  Portions at positions 230-299 (the kept
    tokens in a tile of their own) and 40-109 (kept tokens and window in one tile); heads of 64
    and 128 with pages that divide 128 run on the tcgen05 kernel.  Single tokens in bfloat16 also with
    the context cut into 1, 3, 5 and 12 slices (the kept tokens then fall into a slice of their
    own, share one with the window, or are all there is)."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(3 + hd)
    n, nh, nkv, W, keep, rows, far = 300, 4, 2, 37, 21, 10, 30.0
    keys = torch.randn(n, nkv, hd, generator=g)
    keys[..., -1] = 3.0            # a query along -e_last scores every key far below 0
    keys = (keys / keys.norm(dim=-1, keepdim=True)).to(dt).float()
    values = torch.randn(n, nkv, hd, generator=g).to(dt).float()
    kp, vp, order = _paged(keys, values, page, g, dt)
    rel = torch.randn(rows, nh, generator=g)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0])
    if decode is True:
        # (query position, chosen key, visible)
        cases = [(299, 263, True), (299, 262, False), (299, 20, True), (299, 21, False), (299, 0, True),
                 (299, 15, True), (299, 16, True), (299, 299, True), (299, 288, True), (299, 287, True),
                 (299, 150, False), (57, 21, True), (57, 20, True), (58, 21, False), (36, 0, True),
                 (37, 0, True), (20, 3, True), (0, 0, True), (1, 0, True), (16, 16, True), (47, 32, True),
                 (48, 32, True), (272, 236, True), (272, 235, False)]
        q_pos = torch.tensor([c[0] for c in cases] + [299, 40, 0], dtype=torch.int32)
        chosen = [c[1:] for c in cases] + [None] * 3
    else:
        if decode == "early":
            # a portion whose window still reaches the kept tokens: they and the window's keys share
            # a tile, with keys between them that nobody sees
            q_pos = torch.arange(40, 110, dtype=torch.int32)
            picks = {0: 3, 1: 4, 2: 5, 5: 21, 17: 20, 18: 21, 19: 22, 30: 21, 31: 20, 32: 0, 40: 44, 41: 44, 42: 45,
                     60: 0, 61: 64, 62: 63, 69: 109, 68: 72}
            decode = False
        else:
            q_pos = torch.arange(230, 300, dtype=torch.int32)
            picks = {0: 194, 1: 194, 2: 20, 3: 21, 4: 0, 5: 15, 6: 16, 10: 240, 20: 214, 21: 214, 40: 255, 41: 256,
                     60: 254, 69: 263, 68: 261}
        chosen = []
        for r, p in enumerate(q_pos.tolist()):
            j = picks.get(r)
            chosen.append(None if j is None else (j, (j <= p) and (p - j < W or j < keep)))
        chosen[30] = chosen[31] = "sink"
    q = torch.randn(len(q_pos), nh, hd, generator=g) * 0.1
    for r, c in enumerate(chosen):
        if c == "sink" or (decode and c is None):
            q[r] = 0.0
            q[r, :, -1] = -40.0
        elif c is not None:
            for h in range(nh):
                q[r, h] = keys[c[0], h // (nh // nkv)] * 70.0
    q = q.to(dt)
    gate = torch.randn(len(q_pos), nh * hd + 5, generator=g).to(dt)
    flat = ops.distance_bias_rows(rel.cuda(), far, W)
    options = ops.AttentionOptions(bias_table=flat, sink_values=sink.cuda(), keep_first=keep,
                                   gate=gate.cuda()[:, 2:2 + nh * hd], gate_wide=True)
    want, wts = pg.attend_rows(q.double(), q_pos, keys.double(), values.double(), 1.0, W, keep, sink.double(),
                               rel.double(), far)
    gates = torch.sigmoid(gate[:, 2:2 + nh * hd].double()).view(len(q_pos), nh, hd)
    want = want * gates
    tol = 2e-5 if dtype == "float32" else 2e-2
    rep = nh // nkv
    for splits in ((None, 1, 3, 5, 12) if decode and dtype == "bfloat16" and hd in ops.TILED_HEAD_DIMS else (None,)):
        out = _attend(ops, q.view(len(q_pos), nh * hd).contiguous(), kp, vp, order, q_pos, nh, nkv, hd, page, 1.0, W,
                      options, decode, n, splits).view(len(q_pos), nh, hd)
        for r, c in enumerate(chosen):
            assert (out[r].double() - want[r]).abs().max() < tol * max(1.0, float(want[r].abs().max())), (r, int(q_pos[r]), c)
            if c == "sink" or (decode and c is None):
                assert float(wts[r].sum(-1).max()) < 0.01 and float(out[r].abs().max()) < 0.05
            elif c is not None:
                key, visible = c
                if visible:
                    assert float(wts[r, :, key].min()) > 0.99, "the case does not single out its key"
                    lone = values[key].double().repeat_interleave(rep, 0) * gates[r]
                    assert (out[r].double() - lone).abs().max() < 0.05 * float(values.abs().max())
                else:
                    assert float(wts[r, :, key].max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,P,H,G", [(16, 24, 4, 2), (7, 15, 2, 1), (48, 40, 6, 3), (130, 33, 2, 2), (64, 64, 4, 1)])
def test_state_space_scan_in_two_steps_from_slots_used_again(dtype, N, P, H, G):
    """Three requests of unequal length in one batch, each cut into two steps; the slots hold
    what another request left and are zeroed by hand as the cache manager does at admission.
    Once through the kernel for portions (inputs staged, chunks of 16 fetched ahead: the cuts
    fall inside a chunk, the lengths pass two chunk borders) and once through the kernel for
    single tokens; the two agree bit for bit."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(N + P)
    lengths, cuts, slots = [70, 1, 20], [33, 1, 3], [2, 0, 3]
    ld = H * P + 2 * G * N + 3
    state0 = torch.randn(5, H * N * P, generator=g).cuda()
    for s in slots:
        state0[s].zero_()
    data = [torch.randn(L, ld + H, generator=g).to(dt) for L in lengths]
    a_log, dt_bias, d_skip = (torch.randn(H, generator=g) * 0.5 for _ in range(3))
    def run(most):
        """Both steps with requests of more than ``most`` tokens on the kernel for portions."""
        kept, ops.SSM_DIRECT_MAX_TOKENS = ops.SSM_DIRECT_MAX_TOKENS, most
        state = state0.clone()
        outs = [[] for _ in lengths]
        try:
            for step in range(2):
                parts = [(d[:c] if step == 0 else d[c:]) for d, c in zip(data, cuts)]
                live = [i for i, p in enumerate(parts) if p.shape[0]]
                rows = torch.cat([parts[i] for i in live]).cuda()
                cu = torch.tensor([0] + list(torch.tensor([parts[i].shape[0] for i in live]).cumsum(0)),
                                  dtype=torch.int32)
                ctx = SimpleNamespace(cu_tokens=cu.cuda(), num_seqs=len(live),
                                      slots=torch.tensor([slots[i] for i in live], dtype=torch.int32).cuda())
                xbc = rows[:, :ld].contiguous()
                y = ops.ssm_scan(ctx, xbc, (0, H * P, H * P + G * N), rows[:, ld:], a_log.cuda(), dt_bias.cuda(),
                                 d_skip.cuda(), state, H, G, N, P).cpu()
                for k, i in enumerate(live):
                    outs[i].append(y[cu[k]:cu[k + 1]])
        finally:
            ops.SSM_DIRECT_MAX_TOKENS = kept
        return [torch.cat(o) for o in outs], state.cpu()

    seen = [run(1 << 30), run(0)]
    outs, state = seen[1]
    for a, b in zip(seen[0][0], seen[1][0]):
        assert torch.equal(a, b)
    assert torch.equal(seen[0][1], seen[1][1])
    for i, d in enumerate(data):
        d = d.double()
        want, S = pg.state_space_scan(d[:, :H * P].view(-1, H, P), d[:, H * P:H * P + G * N].view(-1, G, N),
                                      d[:, H * P + G * N:H * P + 2 * G * N].view(-1, G, N), d[:, ld:], dt_bias.double(),
                                      a_log.double(), d_skip.double())
        got = outs[i].double().view(-1, H, P)
        scale = max(1.0, float(want.abs().max()))
        assert (got - want).abs().max() < 2e-5 * scale, (i, float((got - want).abs().max()))
        assert (state[slots[i]].double().view(H, N, P) - S).abs().max() < 2e-5 * max(1.0, float(S.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_before_a_norm_in_parts_and_the_short_convolution(dtype):
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(5)
    y = torch.randn(9, 60, generator=g)
    z = torch.randn(9, 70, generator=g).to(dt)
    w = torch.randn(60, generator=g)
    for parts in (1, 3, 60):
        got = ops.gated_group_rmsnorm(y.cuda(), z.cuda()[:, 4:64], w.cuda(), parts, 1e-5).float().cpu().double()
        v = y.double() * pg.silu(z[:, 4:64].double())
        want = pg.rms_unit(v.view(9, parts, 60 // parts), 1e-5).reshape(9, 60) * w.double()
        assert (got - want).abs().max() < (1e-5 if dtype == "float32" else 3e-2)
    # the convolution: two requests, the second continues from inputs its slot holds; rows of
    # odd sizes with few tokens, and rows that come in 16-byte pieces with many (in bfloat16 a
    # thread then takes eight channels of four tokens, across the border of the two requests)
    for C, width, col0, taps, n0, n1, n2 in [(11, 20, 6, 4, 5, 2, 5), (16, 32, 8, 4, 81, 30, 70),
                                             (24, 40, 16, 3, 62, 3, 66), (8, 16, 8, 2, 1, 70, 64)]:
        x = torch.randn(n0 + n1 + n2, width, generator=g).to(dt)
        cw, cb = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
        state = torch.zeros(3, C * (taps - 1)).cuda()
        ctx = SimpleNamespace(seq_of_token=torch.tensor([0] * n0 + [1] * n1, dtype=torch.int32).cuda(),
                              cu_tokens=torch.tensor([0, n0, n0 + n1], dtype=torch.int32).cuda(),
                              slots=torch.tensor([2, 0], dtype=torch.int32).cuda(), num_seqs=2)
        first = ops.causal_conv_silu(ctx, x[:n0 + n1].cuda(), C, cw.cuda(), state, bias=cb.cuda(), col0=col0).float().cpu()
        ctx2 = SimpleNamespace(seq_of_token=torch.tensor([0] * n2, dtype=torch.int32).cuda(),
                               cu_tokens=torch.tensor([0, n2], dtype=torch.int32).cuda(),
                               slots=torch.tensor([0], dtype=torch.int32).cuda(), num_seqs=1)
        second = ops.causal_conv_silu(ctx2, x[n0 + n1:].cuda(), C, cw.cuda(), state, bias=cb.cuda(), col0=col0).float().cpu()
        xa = x[:n0, col0:col0 + C].double()
        xb = x[n0:, col0:col0 + C].double()
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert (first[:n0].double() - pg.silu(pg.causal_conv(xa, cw.double(), cb.double()))).abs().max() < tol
        wb = pg.silu(pg.causal_conv(xb, cw.double(), cb.double()))
        assert (first[n0:].double() - wb[:n1]).abs().max() < tol and (second.double() - wb[n1:]).abs().max() < tol
    # an activation of one argument, odd sizes and whole 16-byte pieces
    for rows, cols in [(5, 7), (6, 40)]:
        u = torch.randn(rows, cols, generator=g).to(dt)
        got = ops.unary_act(u.cuda(), "relu2").float().cpu().double()
        assert (got - torch.relu(u.double()) ** 2).abs().max() < (1e-6 if dtype == "float32" else 5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("ff", [40, 20])
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_and_experts_against_the_plain_functions(dtype, ff):
    from helios_b200.parts import RoutedExperts

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(ff)
    width, E, top, T = 48, 7, 3, 29
    part = RoutedExperts(width, ff, E, top, router="top_softmax", router_bias=True, weight_on="output",
                         activation="relu2", shared_inner=24)
    t = {}
    for name, spec in part.weight_specs().items():
        x = torch.randn(spec.shape, generator=g) * (0.3 if spec.kind == "matrix" else 1.0)
        t[name] = x.to(dt).float() if spec.kind == "matrix" else x
    h = torch.randn(T, width, generator=g).to(dt).float()
    z = h.double() @ t["router"].double().T + t["router.b"].double()
    srt = z.sort(-1, descending=True).values
    h = h[(srt[:, top - 1] - srt[:, top]) > 0.05]          # tokens whose choice rounding cannot change
    assert h.shape[0] > 10
    part.bind({k: (v.to(dt) if part.weight_specs()[k].kind == "matrix" else v).cuda() for k, v in t.items()})
    got = part.forward(SimpleNamespace(), h.to(dt).cuda()).float().cpu().double()
    w = {"p." + k: v.double() for k, v in t.items()}
    want = pg.routed_feed_forward(h.double(), w, "p.", {"router": {"top": top}, "shared": {"ff": 24}})
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))
    from helios_b200.csrc import ops
    ids, wts = ops.moe_topk(torch.randn(5, 300, generator=g).cuda(), 4, "top_softmax", None,
                            torch.randn(300, generator=torch.Generator().manual_seed(1)).cuda())
    zz = torch.randn(5, 300, generator=torch.Generator().manual_seed(ff)) * 0     # shape only
    assert ids.shape == (5, 4) and abs(float(wts.sum(-1).min()) - 1.0) < 1e-5


# ====================================================================== whole models
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(GB_ALONE) + list(GB_CONFIGS))
def test_whole_prompts_and_the_stream_after_every_layer(gb_folders, name, dtype):
    """Logits at every position of whole prompts (the first tokens of a sequence among them,
    and prompts that pass every window), and the residual stream after every layer."""
    cfg, weights = read_folder(gb_folders[name])
    reqs = _requests(cfg, [1, 2, 3, 41, 130], 100)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.whole(tb, rid, toks)
    core = _core(gb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} whole")
    from helios_b200.engine.batch import StepEntry
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    _, want_layers = pg.model(cfg, w, reqs["q3"])
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
@pytest.mark.parametrize("name", list(GB_CONFIGS))
def test_prefill_then_long_decoding_token_by_token(gb_folders, name, dtype):
    """Most of the prompt in one step, then 70 single tokens (captured decode steps) that pass
    page borders and carry every window over decoded tokens; the recurrent state goes from
    step to step."""
    cfg, weights = read_folder(gb_folders[name])
    reqs = _requests(cfg, [75, 131, 260], 200)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.prefill_then_decode(tb, rid, toks, n_decode=70)
    core = _core(gb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} decode")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(GB_CONFIGS))
def test_portions_of_changing_size_down_to_one_token(gb_folders, name, dtype):
    cfg, weights = read_folder(gb_folders[name])
    reqs = _requests(cfg, [64, 97, 50, 33], 300)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    sizes = [[7], [2, 31, 3, 16, 2, 17], [1, 2, 1, 1, 3, 13, 2, 1, 5], [16, 1, 15, 1]]
    for (rid, toks), sz in zip(reqs.items(), sizes):
        tu.portions(tb, rid, toks, sz)
    core = _core(gb_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} portions")


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(GB_CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(gb_folders, name, dtype, graphs):
    """Nine unequal requests through three slots: portions of some beside single tokens of
    others; every finished request's pages and slot (with the state another left) go to the next."""
    cfg, weights = read_folder(gb_folders[name])
    reqs = _requests(cfg, [40, 23, 77, 18, 52, 31, 66, 20, 45], 400)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=7, max_live=3, decode_tail=10)
    core = _core(gb_folders[name], dtype, tb.live_tokens_peak, max_slots=3, graphs=graphs)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} mixed")
    assert core.cache.num_free_slots == 3 and all(p.num_used == 0 for p in core.cache.pools)


@pytest.mark.gpu
def test_a_batch_gives_each_request_what_it_gets_alone(gb_folders):
    """float32: the same rows bit for bit, alone or beside others, in one step or in portions,
    whatever the slots and pages."""
    from helios_b200.engine.batch import StepEntry

    cfg, _w = read_folder(gb_folders["gb_a"])
    reqs = _requests(cfg, [37, 5, 60], 500)
    core = _core(gb_folders["gb_a"], "float32", 512, max_slots=4)
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
def test_through_trace_run(gb_folders, dtype, tmp_path):
    cfg, weights = read_folder(gb_folders["gb_b"])
    reqs = _requests(cfg, [30, 47, 22, 39, 28], 600)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=3, max_live=4, decode_tail=8)
    got = tu.run_trace_run(gb_folders["gb_b"], dtype, tb, tmp_path / "out", tb.live_tokens_peak, cfg["vocab"])
    tu.check(tb, got, plain, dtype, "gb_b trace_run")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gb_a", "gb_d"])
def test_greedy_generation_through_the_scheduler(gb_folders, name, dtype):
    from helios_b200 import LLM, SamplingParams

    cfg, weights = read_folder(gb_folders[name])
    w = _f64(_bf16(weights) if dtype == "bfloat16" else weights)
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 5, 17, 33, 9, 26)]
    llm = LLM(str(gb_folders[name]), dtype=dtype, kv_cache_bytes=1 << 22, max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(max_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 12
        toks = list(prompt)
        for t in out.token_ids:
            logits = pg.model(cfg, w, toks)[0][-1]
            best = int(torch.argmax(logits))
            if t != best:
                assert dtype == "bfloat16", f"token {t} instead of {best} after {len(toks)} tokens"
                assert float(logits[best] - logits[t]) <= 0.03 * float(logits.abs().max())
            toks.append(t)
