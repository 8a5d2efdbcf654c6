"""Block formats, GGUF reader/writer, resident layouts and the CPU quantised dots."""
import os

import numpy as np
import pytest
import torch

from bloomery_b200.formats import quant as Q
from bloomery_b200.formats.gguf import Gguf, GgufError, GgufWriter, split_paths
from bloomery_b200.formats.resident import from_resident, resident_row_bytes, to_resident
from bloomery_b200.ops import host_ops as H

ALL = list(Q.QUANTIZE)
BAND = {"F32": 1e-7, "F16": 1e-3, "BF16": 8e-3, "Q8_0": 8e-3, "Q6_K": 3e-2, "Q5_K": 5e-2, "Q5_1": 5e-2, "Q5_0": 8e-2,
        "Q4_K": 1e-1, "Q4_1": 1e-1, "Q4_0": 1.5e-1, "Q3_K": 3e-1, "Q2_K": 5e-1, "IQ4_NL": 1.5e-1, "IQ4_XS": 1.5e-1,
        "MXFP4": 2.5e-1, "IQ2_XXS": 6e-1}


@pytest.mark.parametrize("t", ALL)
def test_roundtrip_band(t):
    torch.manual_seed(0)
    w = torch.randn(8, 1024) * 0.02
    b = Q.quantize(w, t)
    assert b.shape == (8, Q.QTYPES[t].row_bytes(1024))
    y = Q.dequantize(b, t, 1024)
    assert ((y - w).abs().max() / w.abs().max()).item() < BAND[t]


@pytest.mark.parametrize("t", ALL)
def test_requantize_is_stable(t):
    """Decoding then re-encoding decoded values reproduces the same decoded values (a valid encoding)."""
    torch.manual_seed(1)
    w = torch.randn(4, 512) * 0.05
    y = Q.dequantize(Q.quantize(w, t), t, 512)
    y2 = Q.dequantize(Q.quantize(y, t), t, 512)
    assert ((y2 - y).abs().max() / y.abs().max()).item() < BAND[t]


def test_scale_min_pack_roundtrip():
    sc = torch.randint(0, 64, (5, 8), dtype=torch.uint8)
    mn = torch.randint(0, 64, (5, 8), dtype=torch.uint8)
    s2, m2 = Q.unpack_scale_min_k4(Q.pack_scale_min_k4(sc, mn))
    assert torch.equal(sc, s2) and torch.equal(mn, m2)


def test_q4k_known_block():
    """A hand-built block decodes by the format's rule: y = d*sc*q - dmin*m."""
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.25).tobytes(), np.uint8)
    sc = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 40]], dtype=torch.uint8)
    mn = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 33]], dtype=torch.uint8)
    blk[4:16] = Q.pack_scale_min_k4(sc, mn)[0].numpy()
    blk[16:] = 0x21  # low nibble 1, high nibble 2
    y = Q.dequantize(torch.from_numpy(blk)[None], "Q4_K", 256)[0]
    for sub in range(8):
        q = 1 if sub % 2 == 0 else 2
        want = 0.5 * int(sc[0, sub]) * q - 0.25 * int(mn[0, sub])
        assert torch.allclose(y[32 * sub:32 * sub + 32], torch.full((32,), want))


def test_gguf_write_read(tmp_path):
    torch.manual_seed(2)
    w = GgufWriter("qwen3moe")
    w.set("qwen3moe.block_count", 2)
    w.set("general.name", "fixture")
    w.set("tokenizer.ggml.tokens", ["a", "b", "c"])
    w.set("some.floats", [0.5, 1.5])
    a = torch.randn(6, 256)
    e = torch.randn(3, 4, 256)
    w.add_quantized("a.weight", a, "Q4_K")
    w.add_quantized("e.weight", e, "Q6_K")
    w.add_f32("n.weight", torch.ones(256))
    path = str(tmp_path / "m.gguf")
    w.write(path)
    with Gguf.open(path) as g:
        assert g.arch == "qwen3moe" and g.arch_get("block_count") == 2
        assert g.get("tokenizer.ggml.tokens") == ["a", "b", "c"]
        assert g.tensors["a.weight"].shape == (6, 256) and g.tensors["a.weight"].ne == (256, 6)
        assert g.tensors["e.weight"].shape == (3, 4, 256)
        assert torch.equal(g.tensor_rows("a.weight").clone(), Q.quantize(a, "Q4_K"))
        assert torch.allclose(g.tensor_f32("n.weight"), torch.ones(256))
        assert g.tensor_f32("e.weight").shape == (3, 4, 256)
        assert len(g.sha256("a.weight")) == 64
    inv = Gguf.inventory(path)
    assert set(inv.tensors) == {"a.weight", "e.weight", "n.weight"}
    inv.close()


def test_gguf_refuses_bad_files(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(GgufError, match="magic"):
        Gguf.open(str(p))
    p.write_bytes(b"GGUF")
    with pytest.raises(GgufError, match="too short"):
        Gguf.open(str(p))


def test_gguf_truncated_data_is_refused(tmp_path):
    w = GgufWriter("llama")
    w.add_quantized("a.weight", torch.randn(4, 256), "Q8_0")
    path = str(tmp_path / "t.gguf")
    w.write(path)
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-40])
    with pytest.raises(GgufError, match="past the end"):
        Gguf.open(path)
    Gguf.inventory(path).close()  # header-only open still lists it


def test_split_paths():
    assert split_paths("/x/m-00002-of-00003.gguf") == [f"/x/m-0000{i}-of-00003.gguf" for i in (1, 2, 3)]
    assert split_paths("/x/m.gguf") == ["/x/m.gguf"]


def test_gguf_split_shards(tmp_path):
    for i, name in ((1, "a.weight"), (2, "b.weight")):
        w = GgufWriter("llama")
        w.set("split.count", 2)
        w.add_quantized(name, torch.randn(2, 256), "Q4_K")
        w.write(str(tmp_path / f"m-0000{i}-of-00002.gguf"))
    with Gguf.open(str(tmp_path / "m-00001-of-00002.gguf")) as g:
        assert set(g.tensors) == {"a.weight", "b.weight"}
        assert g.tensors["b.weight"].shard == 1
        assert g.tensor_f32("b.weight").shape == (2, 256)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K"])
def test_resident_roundtrip_and_host_units(t):
    torch.manual_seed(3)
    K = 1024
    w = torch.randn(24, K) * 0.02
    raw = Q.quantize(w, t)
    res = to_resident(raw, t, K)
    assert res.shape[1] == resident_row_bytes(t, K) and res.shape[1] % 16 == 0
    assert torch.equal(from_resident(res, t, K), raw)
    wd = Q.dequantize(raw, t, K)
    assert torch.equal(H.decode_rows(res, t, K), wd)            # unit decode is exact
    x = torch.randn(3, K)
    x[1, 5] = 40.0                                             # an outlier, as the reference's kernel gates use
    codes, ds = H.act_q8(x)
    c2, ds2 = Q.quantize_act_q8(x)
    assert torch.equal(codes, c2) and torch.allclose(ds, ds2, rtol=1e-6, atol=0)
    xa = Q.dequantize_act_q8(codes, ds)
    ref = (xa.double() @ wd.double().T).float()                 # f64 dot on the same quantised activations
    out = H.gemv(res, t, K, codes, ds)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 1e-5
    assert torch.equal(out, H.gemv(res, t, K, codes, ds))       # bit-identical rerun


def _scalar_decode(raw: bytes, t: str):
    """One block decoded value by value in plain Python integers and floats, straight from the format's definition."""
    import struct
    from bloomery_b200.formats.iq_tables import KVALUES_IQ4NL, KVALUES_MXFP4, iq2xxs_grid
    half = lambda b: struct.unpack("<e", bytes(b))[0]
    out = []
    if t == "IQ4_NL":
        d = half(raw[0:2])
        out = [d * KVALUES_IQ4NL[raw[2 + j] & 15] for j in range(16)] + [d * KVALUES_IQ4NL[raw[2 + j] >> 4] for j in range(16)]
    elif t == "MXFP4":
        e = raw[0]
        d = struct.unpack("<f", struct.pack("<I", (e - 1) << 23 if e >= 2 else (0x00400000 if e == 1 else 0x00200000)))[0]
        out = [d * KVALUES_MXFP4[raw[1 + j] & 15] for j in range(16)] + [d * KVALUES_MXFP4[raw[1 + j] >> 4] for j in range(16)]
    elif t == "IQ4_XS":
        d = half(raw[0:2])
        sh = raw[2] | raw[3] << 8
        for ib in range(8):
            ls = ((raw[4 + ib // 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4)
            dl = d * (ls - 32)
            q = raw[8 + 16 * ib:8 + 16 * ib + 16]
            out += [dl * KVALUES_IQ4NL[b & 15] for b in q] + [dl * KVALUES_IQ4NL[b >> 4] for b in q]
    elif t == "IQ2_XXS":
        d = half(raw[0:2])
        grid = iq2xxs_grid().tolist()
        for ib in range(8):
            w = raw[2 + 8 * ib:2 + 8 * ib + 8]
            aux = w[4] | w[5] << 8 | w[6] << 16 | w[7] << 24
            db = d * (0.5 + (aux >> 28)) * 0.25
            for l in range(4):
                s7 = (aux >> (7 * l)) & 127
                signs = s7 | ((bin(s7).count("1") & 1) << 7)
                out += [db * grid[w[l]][j] * (-1.0 if signs >> j & 1 else 1.0) for j in range(8)]
    return out


@pytest.mark.parametrize("t", ["IQ4_NL", "IQ4_XS", "MXFP4", "IQ2_XXS"])
def test_codebook_types_decode_and_resident_form(t):
    """Random block bytes (every code and scale the format can hold) decode as the format says, value by value; the
    int8-code + f32-scale rows they are loaded as hold exactly those values; the host units dot them."""
    from bloomery_b200.formats.resident import decode_q8_f32, resident_type
    g = torch.Generator().manual_seed(11)
    K = 512
    qt = Q.QTYPES[t]
    raw = torch.randint(0, 256, (5, qt.row_bytes(K)), dtype=torch.uint8, generator=g)
    blk = raw.reshape(5, K // qt.block_values, qt.block_bytes)
    if t == "MXFP4":
        blk[..., 0] = torch.randint(100, 140, blk[..., 0].shape, generator=g).to(torch.uint8)      # scales in f32 range
    else:
        blk[..., 0:2] = Q._f16_bytes(torch.rand(blk.shape[:-1], generator=g) * 0.01 + 1e-3)          # a finite f16 d
    raw = blk.reshape(5, -1).contiguous()
    got = Q.dequantize(raw, t, K)
    want = torch.tensor([sum((_scalar_decode(bytes(b.tolist()), t) for b in row), []) for row in blk], dtype=torch.float32)
    assert torch.equal(got, want)
    res = to_resident(raw, t, K)
    assert resident_type(t) == "Q8_F32" and res.shape[1] == resident_row_bytes("Q8_F32", K)
    assert torch.equal(decode_q8_f32(res, K), got)
    assert torch.equal(H.decode_rows(res, "Q8_F32", K), got)
    x = torch.randn(3, K)
    codes, ds = H.act_q8(x)
    ref = (Q.dequantize_act_q8(codes, ds).double() @ got.double().T).float()
    out = H.gemv(res, "Q8_F32", K, codes, ds)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 1e-5


@pytest.mark.parametrize("t", ["NVFP4", "FP8_B128"])
def test_plane_types_host_units(t):
    from bloomery_b200.formats.resident import quantize_resident
    torch.manual_seed(5)
    K = 1024
    w = torch.randn(24, K) * 0.02
    w[3, 100] = 1.5
    res, wd = quantize_resident(w, t)
    assert res.shape[1] == resident_row_bytes(t, K) and res.shape[1] % 16 == 0
    assert ((wd - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt()).item() < (0.15 if t == "NVFP4" else 0.04)
    assert torch.equal(H.decode_rows(res, t, K), wd)            # unit decode is exact
    x = torch.randn(3, K)
    x[1, 5] = 40.0
    codes, ds = H.act_q8(x)
    ref = (Q.dequantize_act_q8(codes, ds).double() @ wd.double().T).float()
    out = H.gemv(res, t, K, codes, ds)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 1e-5
    assert torch.equal(out, H.gemv(res, t, K, codes, ds))


def test_e4m3_and_plane_refusals():
    from bloomery_b200.formats import planes as P
    c = torch.arange(256, dtype=torch.uint8)
    ref = c.view(torch.float8_e4m3fn).float()
    v = P.e4m3_decode(c)
    ok = ~torch.isnan(ref)
    assert torch.equal(v[ok], ref[ok]) and torch.isnan(v[~ok]).all()
    x = torch.randn(4096) * 60
    assert torch.equal(P.e4m3_encode(x), x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8))
    codes, sc = P.fp8_b128_quantize(torch.randn(130, 256))
    bad = codes.clone(); bad[0, 0] = 0x7F
    with pytest.raises(P.PlaneError):
        P.fp8_b128_resident(bad, sc)
    bads = sc.clone(); bads[0, 0] = float("inf")
    with pytest.raises(P.PlaneError):
        P.fp8_b128_resident(codes, bads)
    with pytest.raises(P.PlaneError):
        P.fp8_b128_resident(codes[:, :192], sc)
    pk, s, t = P.nvfp4_quantize(torch.randn(8, 128))
    with pytest.raises(P.PlaneError):
        P.nvfp4_resident(pk, s[:, :4], t)
    # a compressed-tensors divisor and a ModelOpt multiplier describe the same values
    a = P.nvfp4_resident(pk, s, t)
    assert torch.equal(P.resident_dequantize(a, "NVFP4", 128), P.nvfp4_dequantize(pk, s, t))


def test_safetensors_folder(tmp_path):
    from bloomery_b200.formats import planes as P
    from bloomery_b200.formats import safetensors as S
    torch.manual_seed(6)
    w = torch.randn(130, 256)
    codes, sc = P.fp8_b128_quantize(w)
    pk, s, t = P.nvfp4_quantize(w[:, :128].contiguous())
    tensors = {"a.weight": codes, "a.weight_scale_inv": sc, "b.weight_packed": pk, "b.weight_scale": s,
               "b.weight_global_scale": (1.0 / t).reshape(1), "n.weight": torch.randn(256).bfloat16()}
    tags = {"a.weight": "F8_E4M3", "b.weight_scale": "F8_E4M3"}
    S.write_folder(str(tmp_path / "m"), tensors, {"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}},
                   shards=3, dtypes=tags)
    f = S.Folder(str(tmp_path / "m"))
    assert set(f.names()) == set(tensors) and f.info("a.weight").dtype == "F8_E4M3"
    for n, v in tensors.items():
        assert torch.equal(f.tensor(n), v), n
    assert P.detect_scheme(f.config) == "fp8_b128"
    res, ty, k = P.linear_resident(f, "a", "fp8_b128")
    assert ty == "FP8_B128" and k == 256 and torch.equal(P.resident_dequantize(res, ty, k), P.fp8_b128_dequantize(codes, sc))
    res, ty, k = P.linear_resident(f, "b", "nvfp4_ct")
    assert ty == "NVFP4" and torch.allclose(P.resident_dequantize(res, ty, k), P.nvfp4_dequantize(pk, s, t), rtol=1e-6)
    res, ty, k = P.linear_resident(f, "n", "fp8_b128")        # an unquantised tensor inside a quantised folder
    assert ty == "BF16"
    f.close()
    # refusals: truncated file, entry outside the file, missing shard
    p = str(tmp_path / "one.safetensors")
    S.write_file(p, {"x": torch.arange(10.)})
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:-4])
    with pytest.raises(S.SafetensorsError):
        S.Safetensors(p)
    open(p, "wb").write(blob[:6])
    with pytest.raises(S.SafetensorsError):
        S.Safetensors(p)
    import os
    os.remove(str(tmp_path / "m" / "model-00002-of-00003.safetensors"))
    with pytest.raises(S.SafetensorsError):
        S.Folder(str(tmp_path / "m"))
    with pytest.raises(P.PlaneError):
        P.detect_scheme({"quantization_config": {"quant_method": "awq"}})


def test_host_pool():
    assert H.pool_size() >= 1


def test_cpu_expert_leg_matches_oracle():
    """blh_moe_experts (C++ pool, unit dots) against the fp32 restatement on the same q8 inputs."""
    import ctypes
    from bloomery_b200.formats.resident import WT
    from bloomery_b200.ops._lib import host
    torch.manual_seed(5)
    H, I, E, k, M = 512, 256, 6, 3, 2
    gate = torch.randn(E, I, H) * 0.05; up = torch.randn(E, I, H) * 0.05; down = torch.randn(E, H, I) * 0.05
    def res(w, t):
        raw = Q.quantize(w.reshape(-1, w.shape[-1]), t)
        return to_resident(raw, t, w.shape[-1]).contiguous(), Q.dequantize(raw, t, w.shape[-1]).reshape(w.shape)
    gr, gd = res(gate, "Q4_K"); ur, ud = res(up, "Q4_K"); dr, dd = res(down, "Q6_K")
    x = torch.randn(M, H)
    codes, ds = H_act(x)
    ids = torch.tensor([[0, 3, -1], [5, 1, 2]], dtype=torch.int32)
    wts = torch.rand(M, k)
    out = torch.zeros(M, H)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = host().blh_moe_experts(M, H, I, E, k, vp(ids), vp(wts), vp(codes), vp(ds), vp(gr), vp(ur), vp(dr), WT["Q4_K"], WT["Q6_K"], vp(out))
    assert rc == 0
    xa = Q.dequantize_act_q8(codes, ds).double()
    ref = torch.zeros(M, H, dtype=torch.float64)
    for m in range(M):
        for j in range(k):
            e = int(ids[m, j])
            if e < 0:
                continue
            a = (torch.nn.functional.silu(xa[m] @ gd[e].double().T) * (xa[m] @ ud[e].double().T)).float()
            ac, ads = Q.quantize_act_q8(a[None])
            ref[m] += wts[m, j].double() * (Q.dequantize_act_q8(ac, ads)[0].double() @ dd[e].double().T)
    assert ((out.double() - ref).abs().max() / ref.abs().max()).item() < 1e-3


def H_act(x):
    return H.act_q8(x)


def test_residency_rule_is_deterministic_and_bounded():
    from bloomery_b200.runtime.residency import ResidencyRule
    def run():
        r = ResidencyRule(2, 8, [[0, 1, 2], [0, 1, 2]], every=4, cap=3, margin=3.0, min_count=2, decay=0.9)
        log = []
        for step in range(12):
            r.observe(0, [0, 0, 0, 5, 4, 0, 0, 1]); r.observe(1, [1, 1, 1, 0, 0, 0, 0, 0])
            if r.kept(2):
                log.append([(f.layer, f.newcomer, f.victim) for f in r.decide()])
        return log, [sorted(s) for s in r.on_card]
    a, b = run(), run()
    assert a == b                                            # same history => same map
    log, on = a
    assert on[1] == [0, 1, 2] and 3 in on[0] and 4 in on[0]   # the hot ones were promoted, layer 1 untouched
    assert all(len(f) <= 3 for f in log)


@pytest.mark.parametrize("scheme", ["fp8_b128", "nvfp4_modelopt", "nvfp4_ct", "plain"])
def test_checkpoint_folder_opens_as_model(scheme, tmp_path):
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.cpu_ref import CpuModel
    from bloomery_b200.models.spec import tiny_qwen3moe
    spec = tiny_qwen3moe()
    spec.vocab = 1024
    W.write_folder(spec, str(tmp_path / "m"), scheme, seed=1, shards=3)
    sp, w, folder = W.open_model(str(tmp_path / "m"), "cpu")
    assert (sp.n_layer, sp.hidden, sp.n_expert, sp.n_used, sp.head_dim) == (4, 512, 16, 4, 64)
    want = {"fp8_b128": "FP8_B128", "nvfp4_modelopt": "NVFP4", "nvfp4_ct": "NVFP4", "plain": "BF16"}[scheme]
    assert w.q["blk.1.ffn_gate_exps.weight"].qtype == want and w.q["blk.1.ffn_gate_exps.weight"].data.shape[0] == 16
    assert w.q["token_embd.weight"].qtype == "BF16" and w.f["blk.0.attn_norm.weight"].dtype == torch.float32
    out = CpuModel(w).forward(torch.arange(6))
    assert out.shape == (6, 1024) and bool(torch.isfinite(out).all())


def test_deepseek_shape_roundtrips_and_oracle_runs(tmp_path):
    """The MLA / shared-expert / sigmoid-router plan survives GGUF and config.json, and the oracle's
    incremental decode equals its one-shot forward."""
    import dataclasses
    from bloomery_b200.formats.gguf import Gguf
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.cpu_ref import CpuModel
    from bloomery_b200.models.spec import ModelSpec, tiny_deepseek
    spec = tiny_deepseek()
    spec.vocab = 512
    items = list(W.synth_tensors(spec, "cpu", seed=2))
    W.write_gguf(spec, iter(items), str(tmp_path / "d.gguf"))
    sp2, w2, g = W.load_gguf(str(tmp_path / "d.gguf"), "cpu")
    keys = ("n_layer", "hidden", "n_q", "q_lora", "kv_lora", "rope_dim", "nope_dim", "v_dim", "first_dense", "n_shared",
            "router_mode", "router_renorm", "n_group", "topk_group", "n_expert", "n_used", "rope_yarn_factor",
            "rope_yarn_orig_ctx")
    for k in keys:
        assert getattr(sp2, k) == getattr(spec, k), k
    assert abs(sp2.router_scale - spec.router_scale) < 1e-6 and abs(sp2.rope_mscale_all_dim - 1.0) < 1e-6
    sp3 = ModelSpec.from_hf_config(spec.to_hf_config())
    for k in keys:
        assert getattr(sp3, k) == getattr(spec, k), k
    assert w2.f["blk.0.attn_k_b.weight"].shape == (8, 128, 512)
    m = CpuModel(w2)
    toks = torch.arange(7) * 31 % 512
    full = m.forward(toks)
    m.reset()
    inc = torch.cat([m.forward(toks[:4]), m.forward(toks[4:])])
    # batched and single-row products round differently, which can flip a q8 activation code
    assert ((full - inc).abs().max() / full.abs().max()).item() < 2e-2


@pytest.mark.parametrize("t", ["Q4_K", "Q6_K", "Q8_0"])
def test_vector_row_dots_agree_with_the_scalar_units(t):
    """The AVX2 paths of the host expert leg against the scalar mirror of the device units and an f64 dot."""
    import ctypes
    from bloomery_b200.formats.resident import WT
    from bloomery_b200.ops._lib import host, p as vp
    torch.manual_seed(11)
    K = 2048
    w = torch.randn(40, K) * 0.02
    w[3, 7] = 0.9
    raw = Q.quantize(w, t)
    res = to_resident(raw, t, K)
    wd = Q.dequantize(raw, t, K)
    x = torch.randn(1, K)
    x[0, 100] = -25.0
    codes, ds = H.act_q8(x)
    ref = (Q.dequantize_act_q8(codes, ds).double() @ wd.double().T)[0]
    scalar = H.gemv(res, t, K, codes, ds)[0]
    served = 0
    for r in range(40):
        o = ctypes.c_float()
        served += host().blh_row_dot_fast(WT[t], vp(res[r]), K, vp(codes), vp(ds), ctypes.byref(o))
        assert abs(o.value - float(ref[r])) <= 1e-5 * float(ref.abs().max())
        assert abs(o.value - float(scalar[r])) <= 2e-6 * float(ref.abs().max())
    assert served in (0, 40)            # 0 on a host without AVX2: the scalar units serve every type


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "IQ4_XS"])
def test_vnni_row_dots_agree_with_the_scalar_units(t):
    """The AVX-512 VNNI row dots (picked at run time where the CPU has them) against the f64 reference and the scalar
    units; IQ4_XS stands for the int8-code + f32-scale rows every code-book type is loaded as."""
    import ctypes
    from bloomery_b200.formats.resident import WT, resident_type
    from bloomery_b200.ops._lib import host, p as vp
    torch.manual_seed(12)
    K = 2048
    w = torch.randn(33, K) * 0.02
    w[5, 9] = -0.8
    raw = Q.quantize(w, t)
    res = to_resident(raw, t, K)
    rt = resident_type(t)
    wd = Q.dequantize(raw, t, K)
    x = torch.randn(1, K)
    x[0, 77] = 31.0
    codes, ds = H.act_q8(x)
    ref = (Q.dequantize_act_q8(codes, ds).double() @ wd.double().T)[0]
    served = 0
    for r in range(33):
        o = ctypes.c_float()
        served += host().blh_row_dot_vnni(WT[rt], vp(res[r]), K, vp(codes), vp(ds), ctypes.byref(o))
        if served:
            assert abs(o.value - float(ref[r])) <= 1e-5 * float(ref.abs().max()), (r, o.value, float(ref[r]))
    assert served == (33 if host().blh_cpu_has_vnni() else 0)
    # the pool's gemv takes the same path: its rows agree with the reference too
    out = H.gemv(res, rt, K, codes, ds)[0]
    assert ((out - ref.float()).abs().max() / ref.abs().max()).item() < 1e-5


def _scale_bytes(rows, cols, seed, spread=3, outliers=0.02):
    """E4M3-like scale bytes: a row's bytes sit in a narrow window, a few far outside it."""
    rng = np.random.default_rng(seed)
    centre = rng.integers(40, 200, size=(rows, 1))
    sc = np.clip(centre + rng.integers(-spread, spread + 9, size=(rows, cols)), 0, 255)
    far = rng.random((rows, cols)) < outliers
    sc[far] = rng.integers(0, 256, size=int(far.sum()))
    return sc.astype(np.uint8)


@pytest.mark.parametrize("rows,cols", [(32, 8), (64, 7), (160, 10), (4224, 6)])
def test_compressed_nvfp4_scales_decode_to_the_bytes_they_encode(rows, cols):
    from bloomery_b200.formats import csf
    sc = _scale_bytes(rows, cols, rows + cols)
    if cols % 2 == 0:
        parts = csf.encode_csf(sc)
        assert parts["nvfp4_csf_fixed"].shape == (rows // 16, 16 * (1 + cols // 2))
        assert 0 < parts["nvfp4_csf_exceptions"].size < rows * cols // 8          # the window holds most bytes
        got = csf.decode_csf("s", parts["nvfp4_csf_fixed"], parts["nvfp4_csf_exceptions"], rows, cols)
        assert np.array_equal(got, sc)
    p32 = csf.encode_csf32(sc)
    blocks = rows // 32 * ((cols + 1) // 2)
    tiles = -(-(rows // 32) // 4) * -(-((cols + 1) // 2) // 2)
    assert p32["csf32_offsets"].size == blocks + -(-tiles // 32) and p32["csf32_codes"].size == rows * cols // 2
    got = csf.decode_csf32("s", p32["csf32_bases"], p32["csf32_codes"], p32["csf32_page_bases"], p32["csf32_offsets"],
                           p32["csf32_exceptions"], rows, cols)
    assert np.array_equal(got, sc)
    if rows == 4224:
        assert p32["csf32_page_bases"].size > 1 and int(p32["csf32_page_bases"][1]) > 0     # more than one page of records


def test_compressed_scales_breaking_a_rule_are_refused_by_name():
    from bloomery_b200.formats import csf
    sc = _scale_bytes(64, 8, 1)
    a = csf.encode_csf(sc)
    fixed, exc = a["nvfp4_csf_fixed"].copy(), a["nvfp4_csf_exceptions"].copy()
    with pytest.raises(csf.CsfError, match="slabs"):
        csf.decode_csf("s", fixed.reshape(-1)[:-1], exc, 64, 8)
    with pytest.raises(csf.CsfError, match="multiple of 16"):
        csf.decode_csf("s", fixed, exc, 60, 8)
    bad = fixed.copy(); bad[1, 3] = 241
    with pytest.raises(csf.CsfError, match="row 19 base 241"):
        csf.decode_csf("s", bad, exc, 64, 8)
    with pytest.raises(csf.CsfError, match="increasing"):
        csf.decode_csf("s", fixed, exc[::-1].copy(), 64, 8)
    with pytest.raises(csf.CsfError, match="below 512"):
        csf.decode_csf("s", fixed, np.asarray([600], dtype=np.uint32), 64, 8)
    b = csf.encode_csf32(sc)
    args = lambda **kw: [kw.get(k, b[k]) for k in ("csf32_bases", "csf32_codes", "csf32_page_bases", "csf32_offsets", "csf32_exceptions")]  # noqa: E731
    with pytest.raises(csf.CsfError, match="offsets hold"):
        csf.decode_csf32("s", *args(csf32_offsets=b["csf32_offsets"][:-1]), 64, 8)
    with pytest.raises(csf.CsfError, match="page 0: base 2"):
        csf.decode_csf32("s", *args(csf32_page_bases=np.asarray([2], dtype=np.uint32)), 64, 8)
    off = b["csf32_offsets"].copy(); off[-1] += 1
    with pytest.raises(csf.CsfError, match="prefixes|records"):
        csf.decode_csf32("s", *args(csf32_offsets=off), 64, 8)
    if b["csf32_exceptions"].size:
        recs = b["csf32_exceptions"].copy(); recs[0] = (recs[0] & 0xFF00) | 200          # place 200: row 100 of a 32-row block
        with pytest.raises(csf.CsfError, match="outside its 32"):
            csf.decode_csf32("s", *args(csf32_exceptions=recs), 64, 8)
    with pytest.raises(csf.CsfError, match="records"):
        csf.decode_csf32("s", *args(csf32_exceptions=np.append(b["csf32_exceptions"], np.uint16(5))), 64, 8)


@pytest.mark.parametrize("enc", ["csf", "csf_32x2_v1"])
def test_modelopt_checkpoint_with_compressed_scales_loads_like_the_plain_one(tmp_path, enc):
    from bloomery_b200.formats import csf
    from bloomery_b200.formats import planes as P
    from bloomery_b200.formats import safetensors as S
    torch.manual_seed(8)
    w = torch.randn(64, 256)
    pk, s, t = P.nvfp4_quantize(w)
    parts = (csf.encode_csf if enc == "csf" else csf.encode_csf32)(s.view(torch.uint8).numpy())
    tensors = {"a.weight": pk, "a.weight_scale_2": t.reshape(1)}
    tags = {}
    for suffix, arr in parts.items():
        signed = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}.get(arr.dtype)
        tensors[f"a.weight_scale.{suffix}"] = torch.from_numpy(arr.view(signed) if signed else arr.copy())
        if signed:
            tags[f"a.weight_scale.{suffix}"] = "U16" if arr.dtype == np.uint16 else "U32"
    S.write_folder(str(tmp_path / "m"), tensors, {"quantization_config": {"quant_method": "modelopt", "quant_algo": "NVFP4"}},
                   dtypes=tags)
    f = S.Folder(str(tmp_path / "m"))
    res, ty, k = P.linear_resident(f, "a", "nvfp4_modelopt")
    assert ty == "NVFP4" and k == 256
    assert torch.equal(res, P.nvfp4_resident(pk, s, t))
    f.close()


def test_mxfp8_checkpoint_loads_as_exact_bf16_rows(tmp_path):
    from bloomery_b200.formats import planes as P
    from bloomery_b200.formats import safetensors as S
    g = torch.Generator().manual_seed(9)
    codes = torch.randint(0, 256, (48, 128), generator=g, dtype=torch.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3A                               # no NaN codes
    scales = torch.randint(110, 140, (48, 4), generator=g, dtype=torch.uint8)
    want = (P.e4m3_decode(codes).reshape(48, 4, 32).double() * torch.exp2(scales.double() - 127)[:, :, None]).reshape(48, 128)
    got = P.mxfp8_dequantize(codes, scales)
    assert got.dtype == torch.bfloat16 and torch.equal(got.double(), want)          # exact: nothing is rounded
    S.write_folder(str(tmp_path / "m"), {"a.weight": codes, "a.weight_scale": scales, "n.weight": torch.randn(16, 128).bfloat16()},
                   {"quantization_config": {"quant_method": "mxfp8"}}, dtypes={"a.weight": "F8_E4M3", "a.weight_scale": "F8_E8M0"})
    f = S.Folder(str(tmp_path / "m"))
    assert P.detect_scheme(f.config) == "mxfp8"
    res, ty, k = P.linear_resident(f, "a", "mxfp8")
    assert ty == "BF16" and k == 128 and torch.equal(res.view(torch.bfloat16).double(), want)
    assert P.linear_resident(f, "n", "mxfp8")[1] == "BF16"
    f.close()
    with pytest.raises(P.PlaneError, match="255"):
        P.mxfp8_dequantize(codes, torch.full((48, 4), 255, dtype=torch.uint8))


def test_packed_mxfp4_checkpoint_loads_as_exact_code_rows(tmp_path):
    from bloomery_b200.formats import planes as P
    from bloomery_b200.formats import safetensors as S
    from bloomery_b200.formats.resident import decode_q8_f32
    g = torch.Generator().manual_seed(10)
    packed = torch.randint(0, 256, (24, 64), generator=g, dtype=torch.uint8)               # 128 values a row
    scales = torch.randint(118, 134, (24, 4), generator=g, dtype=torch.uint8)
    mag = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float64)
    vals = torch.stack([mag[(packed & 15).long()], mag[(packed >> 4).long()]], dim=-1).reshape(24, 4, 32)
    want = (vals * torch.exp2(scales.double() - 127)[:, :, None]).reshape(24, 128)
    S.write_folder(str(tmp_path / "m"), {"a.weight_packed": packed, "a.weight_scale": scales},
                   {"quantization_config": {"quant_method": "compressed-tensors", "format": "mxfp4-pack-quantized"}})
    f = S.Folder(str(tmp_path / "m"))
    assert P.detect_scheme(f.config) == "mxfp4_ct"
    res, ty, k = P.linear_resident(f, "a", "mxfp4_ct")
    assert ty == "Q8_F32" and k == 128
    assert torch.equal(decode_q8_f32(res, k).double(), want)
    f.close()


@pytest.mark.parametrize("t,lo,hi", [("FP8_B128", 128, 384), ("FP8_B128", 0, 512), ("NVFP4", 48, 304), ("NVFP4", 256, 512)])
def test_plane_rows_slice_by_columns(t, lo, hi):
    from bloomery_b200.formats import planes as P
    from bloomery_b200.formats.resident import quantize_resident, resident_row_bytes
    torch.manual_seed(12)
    res, vals = quantize_resident(torch.randn(20, 512) * 0.1, t)
    cut = P.resident_k_slice(res, t, 512, lo, hi)
    assert cut.shape == (20, resident_row_bytes(t, hi - lo))
    assert torch.equal(P.resident_dequantize(cut, t, hi - lo), vals[:, lo:hi])
    with pytest.raises(P.PlaneError):
        P.resident_k_slice(res, t, 512, lo + 8, hi)


def test_fp8_model_shards_by_heads_experts_and_widths():
    """``shard_items`` on a DeepSeek-shaped FP8 stream: every rank's share decodes to the matching slice of the whole."""
    from bloomery_b200.models.spec import tiny_deepseek
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.parallel.sharded import local_spec, shard_items
    spec = tiny_deepseek()
    items = list(synth_tensors(spec, "cpu", seed=4, mix="FP8_B128"))
    full = Weights.from_items(spec, iter(items), "cpu")
    for rank in range(2):
        w = Weights.from_items(local_spec(spec, 2, attn=False), shard_items(iter(items), spec, rank, 2, attn=False), "cpu")
        d_full, d = full.dequant("blk.0.ffn_down.weight"), w.dequant("blk.0.ffn_down.weight")
        half = d_full.shape[1] // 2
        assert torch.equal(d, d_full[:, rank * half:(rank + 1) * half])                      # dense width: columns
        g_full, g = full.dequant("blk.1.ffn_gate_shexp.weight"), w.dequant("blk.1.ffn_gate_shexp.weight")
        assert torch.equal(g, g_full[rank * g.shape[0]:(rank + 1) * g.shape[0]])             # shared expert: rows
        s_full, s_ = full.dequant("blk.1.ffn_down_shexp.weight"), w.dequant("blk.1.ffn_down_shexp.weight")
        assert torch.equal(s_, s_full[:, rank * s_.shape[1]:(rank + 1) * s_.shape[1]])
        e_full, e = full.dequant("blk.2.ffn_up_exps.weight"), w.dequant("blk.2.ffn_up_exps.weight")
        assert torch.equal(e, e_full[rank * 8:(rank + 1) * 8])                               # experts: by index
        assert torch.equal(w.dequant("blk.1.attn_output.weight"), full.dequant("blk.1.attn_output.weight"))   # attention whole
