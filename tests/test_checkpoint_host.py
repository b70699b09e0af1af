"""The checkpoint reader without a GPU: synthetic checkpoints written here in the safetensors layout, in the
style of berth's crates/berth-exl3/tests/synthetic.rs (groups linears and unpacks signs, padded header, sharded
index with total_size, the rejections and the substrings they carry), and the unpack_signs known answers of
crates/berth-exl3/src/signs.rs:52-91 checked against the oracle's restatement."""
import json
import os
import struct

import numpy as np
import pytest

from berth_b200 import checkpoint
from berth_b200.checkpoint import Checkpoint, CheckpointError
from berth_b200.kernels import Codebook

_NP = {"I16": np.int16, "F16": np.float16, "I32": np.int32, "F32": np.float32, "BF16": np.uint16, "U8": np.uint8}


def write_safetensors(path, tensors, pad=0, metadata=None):
    """tensors: list of (name, dtype name, shape, bytes).  Returns the data bytes written."""
    header, blob, off = {}, b"", 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dt, shape, data in tensors:
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(data)]}
        blob += data
        off += len(data)
    text = json.dumps(header).encode() + b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + blob)
    return off


def t(name, dt, shape, fill=None):
    n = int(np.prod(shape)) if len(shape) else 1
    arr = np.zeros(n, _NP[dt]) if fill is None else np.asarray(fill, _NP[dt]).reshape(-1)
    assert arr.size == n
    return (name, dt, tuple(shape), arr.tobytes())


def linear_parts(prefix, last, marker=None, packed_in=False, packed_out=False, k_tiles=2, n_tiles=3, su=None, sv=None):
    parts = [t(f"{prefix}.trellis", "I16", (k_tiles, n_tiles, last))]
    parts.append(t(f"{prefix}.su", "I16", (k_tiles,), su) if packed_in else t(f"{prefix}.suh", "F16", (k_tiles * 16,)))
    parts.append(t(f"{prefix}.sv", "I16", (n_tiles,), sv) if packed_out else t(f"{prefix}.svh", "F16", (n_tiles * 16,)))
    if marker:
        parts.append(t(f"{prefix}.{marker}", "I32", ()))
    return parts


def open_single(tmp_path, tensors, **kw):
    write_safetensors(tmp_path / "model.safetensors", tensors, **kw)
    return Checkpoint.open(str(tmp_path))


def test_groups_linears_and_unpacks_signs(tmp_path):
    tensors = (linear_parts("model.layers.0.mlp.gate_proj", 64, "mul1") +
               linear_parts("model.layers.0.mlp.down_proj", 48, "mcg", packed_in=True, packed_out=True, su=[1, -32768], sv=[0, 3, -1]) +
               linear_parts("model.layers.0.mlp.up_proj", 40, "mul1") +        # 2.5 bits per weight
               linear_parts("lm_head", 96) +
               [t("model.layers.0.mlp.down_proj.suh", "F16", (32,), np.full(32, 2.0)),     # unpacked wins over packed
                t("model.norm.weight", "BF16", (8,)), t("model.layers.0.mlp.gate.weight", "F16", (4, 32))])
    with open_single(tmp_path, tensors, metadata={"format": "pt"}) as ck:
        lins = ck.linears()
        assert [l.prefix for l in lins] == sorted(l.prefix for l in lins) and len(lins) == 4
        by = {l.prefix: l for l in lins}
        g, d, u, h = (by[p] for p in ("model.layers.0.mlp.gate_proj", "model.layers.0.mlp.down_proj", "model.layers.0.mlp.up_proj", "lm_head"))
        assert (g.k, g.codebook, g.input_packed, g.in_features, g.out_features) == (4.0, Codebook.Mul1, False, 32, 48)
        assert (d.k, d.codebook, d.input_packed, d.output_packed) == (3.0, Codebook.Mcg, False, True)
        assert d.input_scale.name.endswith(".suh")
        assert (u.k, u.codebook) == (2.5, Codebook.Mul1)
        assert (h.k, h.codebook, h.bias) == (6.0, Codebook.Default, None)
        # the packed su of down_proj stays in the index and is not an "other" tensor
        assert ck.tensor("model.layers.0.mlp.down_proj.su").dtype == "I16"
        assert [o.name for o in ck.other_tensors()] == ["model.layers.0.mlp.gate.weight", "model.norm.weight"]
        assert len(ck.tensors()) == len(tensors)
        sv = ck.scale_f16("model.layers.0.mlp.down_proj", True)
        assert sv.shape == (48,) and (sv[:16] == 0x3C00).all()
        assert list(sv[16:20]) == [0xBC00, 0xBC00, 0x3C00, 0x3C00] and (sv[32:] == 0xBC00).all()
        assert (ck.scale_f16("model.layers.0.mlp.down_proj", False).view(np.float16) == 2.0).all()
        w = ck.load_linear("lm_head")
        assert w["trellis"].shape == (2, 3, 96) and w["trellis"].dtype == np.uint16 and (w["bits"], w["cb"]) == (6, 0)
        with pytest.raises(CheckpointError, match="half-integer"):
            ck.load_linear("model.layers.0.mlp.up_proj")
        with pytest.raises(CheckpointError, match="no such"):
            ck.linear("model.layers.0.mlp")
        # the C entry point refuses a destination of the wrong size
        from berth_b200 import _lib
        buf = np.zeros(4, np.uint8)
        assert _lib.lib().berth_ckpt_read(ck._h, b"model.norm.weight", buf.ctypes.data, 4) == -1
        assert b"destination" in _lib.lib().berth_ckpt_last_error()


def test_padded_header_and_data_round_trip(tmp_path):
    data = np.arange(2 * 3 * 64, dtype=np.int16) - 77
    tensors = [t("a.proj.trellis", "I16", (2, 3, 64), data), t("a.proj.suh", "F16", (32,), np.linspace(-1, 1, 32)),
               t("a.proj.svh", "F16", (48,), np.ones(48))]
    with open_single(tmp_path, tensors, pad=37) as ck:
        assert (ck.read("a.proj.trellis").reshape(-1) == data).all()
        assert ck.tensor("a.proj.suh").shape == (32,)
        assert (ck.load_linear("a.proj")["suh"].view(np.float16) == np.linspace(-1, 1, 32).astype(np.float16)).all()


def test_sharded_index_checks_total_size(tmp_path):
    a, b = linear_parts("a.proj", 16, "mul1"), linear_parts("b.proj", 32)
    na = write_safetensors(tmp_path / "model-00001-of-00002.safetensors", a)
    nb = write_safetensors(tmp_path / "model-00002-of-00002.safetensors", b)
    wm = {name: "model-00001-of-00002.safetensors" for name, *_ in a}
    wm.update({name: "model-00002-of-00002.safetensors" for name, *_ in b})
    idx = tmp_path / "model.safetensors.index.json"
    idx.write_text(json.dumps({"metadata": {"total_size": na + nb}, "weight_map": wm}))
    with Checkpoint.open(str(tmp_path)) as ck:
        assert [l.prefix for l in ck.linears()] == ["a.proj", "b.proj"]
        assert ck.tensor("b.proj.trellis").shard.endswith("00002-of-00002.safetensors")
    idx.write_text(json.dumps({"metadata": {"total_size": 1}, "weight_map": wm}))
    with pytest.raises(CheckpointError, match="total_size"):
        Checkpoint.open(str(tmp_path))
    idx.write_text(json.dumps({"weight_map": {"missing.trellis": "model-00001-of-00002.safetensors"}}))
    with pytest.raises(CheckpointError, match="a.proj|missing.trellis"):
        Checkpoint.open(str(tmp_path))
    idx.write_text(json.dumps({"weight_map": {"a.proj.trellis": "../outside.safetensors"}}))
    with pytest.raises(CheckpointError, match="weight_map"):
        Checkpoint.open(str(tmp_path))


@pytest.mark.parametrize("tensors,needle", [
    (linear_parts("h.proj", 24, "mcg"), "mul1"),
    (linear_parts("h.proj", 64, "mul1") + [t("h.proj.mcg", "I32", ())], "both mcg and mul1"),
    (linear_parts("h.proj", 144, "mul1"), "1..=8"),
    (linear_parts("h.proj", 72, "mul1"), "4.5"),
    (linear_parts("h.proj", 20, "mul1"), r"16\*K"),
    ([p for p in linear_parts("h.proj", 64, "mul1") if not p[0].endswith(("suh", "svh"))], "suh"),
    ([t("h.proj.trellis", "I16", (16,)), t("h.proj.suh", "F16", (16,)), t("h.proj.svh", "F16", (16,))], "rank 3"),
    ([t("h.proj.trellis", "F16", (1, 1, 16)), t("h.proj.suh", "F16", (16,)), t("h.proj.svh", "F16", (16,))], "expected I16"),
    (linear_parts("h.proj", 64) + [t("h.proj.bias", "I32", (48,))], "float bias"),
    ([t(".trellis", "I16", (1, 1, 16))], "empty linear prefix"),
])
def test_rejects_bad_linears(tmp_path, tensors, needle):
    with pytest.raises(CheckpointError, match=needle):
        open_single(tmp_path, tensors)


def _write_raw(path, header: str, data: bytes):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header.encode() + data)


def test_rejects_bad_headers(tmp_path):
    p = tmp_path / "model.safetensors"
    _write_raw(p, '{"h.proj.trellis":{"dtype":"I16","shape":[1],"data_offsets":[0,4]}}', b"\0\0\0\0")
    with pytest.raises(CheckpointError, match="h.proj.trellis.*span"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '{"h.proj.trellis":{"dtype":"I16","shape":[1],"data_offsets":[0,2]}}', b"")
    with pytest.raises(CheckpointError, match="h.proj.trellis.*extends"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '{"x":{"dtype":"I17","shape":[1],"data_offsets":[0,2]}}', b"\0\0")
    with pytest.raises(CheckpointError, match="unknown safetensors dtype"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '{"x":{"dtype":"I16","shape":[1],"data_offsets":[2,0]}}', b"\0\0")
    with pytest.raises(CheckpointError, match="before start"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '{"x":{"dtype":"I16","shape":[1],"data_offsets":[0,2]},"x":{"dtype":"I16","shape":[1],"data_offsets":[0,2]}}', b"\0\0")
    with pytest.raises(CheckpointError, match="duplicated"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '[1, 2]', b"")
    with pytest.raises(CheckpointError, match="not a JSON object"):
        Checkpoint.open(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(CheckpointError, match="header length"):
        Checkpoint.open(str(tmp_path))
    _write_raw(p, '{"x":{"dtype":"I16","shape":[1],"data_offsets":[0,2]', b"\0\0")
    with pytest.raises(CheckpointError, match="JSON"):
        Checkpoint.open(str(tmp_path))


def test_missing_checkpoint_names_the_reason(tmp_path):
    with pytest.raises(CheckpointError, match="model.safetensors"):
        Checkpoint.open(str(tmp_path))
    with pytest.raises(CheckpointError, match="not a checkpoint directory"):
        Checkpoint.open(str(tmp_path / "nope"))


def test_unpack_signs_known_answers():
    """crates/berth-exl3/src/signs.rs:52-91, and the oracle's restatement on random words."""
    one, neg = 0x3C00, 0xBC00
    s = checkpoint.unpack_signs(struct.pack("<H", 1))
    assert s.shape == (16,) and s[0] == neg and (s[1:] == one).all()
    s = checkpoint.unpack_signs(struct.pack("<H", 0x8000))
    assert s[15] == neg and (s[:15] == one).all()
    assert (checkpoint.unpack_signs(struct.pack("<H", 0)) == one).all()
    s = checkpoint.unpack_signs(np.array([0x0001, 0x0002], np.uint16))
    assert s.shape == (32,) and s[0] == neg and s[17] == neg and (s == neg).sum() == 2
    assert checkpoint.unpack_signs(b"").shape == (0,)
    with pytest.raises(CheckpointError, match="multiple of 2"):
        checkpoint.unpack_signs(b"\x01")
    from oracle import exl3_oracle
    words = np.random.default_rng(7).integers(0, 65536, 257).astype(np.uint16)
    assert (checkpoint.unpack_signs(words) == exl3_oracle.unpack_signs(words)).all()


def test_load_experts_stacks_the_per_expert_tensors(tmp_path):
    tensors = []
    for e in range(3):
        for proj, (kt, nt) in (("gate", (2, 1)), ("up", (2, 1)), ("down", (1, 2))):
            tr = np.full(kt * nt * 64, 100 * e + len(proj), np.int16)
            tensors += [t(f"m.mlp.experts.{e}.{proj}_proj.trellis", "I16", (kt, nt, 64), tr),
                        t(f"m.mlp.experts.{e}.{proj}_proj.su", "I16", (kt,), [e] * kt),
                        t(f"m.mlp.experts.{e}.{proj}_proj.svh", "F16", (nt * 16,), np.full(nt * 16, e + 1.0)),
                        t(f"m.mlp.experts.{e}.{proj}_proj.mul1", "I32", ())]
    with open_single(tmp_path, tensors) as ck:
        w = ck.load_experts("m.mlp", 3)
        assert w["gate_trellis"].shape == (3, 2, 1, 64) and w["down_trellis"].shape == (3, 1, 2, 64)
        assert (w["bits"], w["cb"], w["n_experts"]) == (4, 2, 3)
        assert (w["up_trellis"][2] == 202).all() and (w["down_svh"][1].view(np.float16) == 2.0).all()
        assert w["gate_suh"].shape == (3, 32) and w["gate_suh"][1][0] == 0xBC00 and w["gate_suh"][2][1] == 0xBC00
        with pytest.raises(CheckpointError, match="no such linear"):
            ck.load_experts("m.mlp", 4)
