"""Seeded mutation runs over the two host-side parsers of untrusted files: ``config.json`` and the safetensors header.
Every input must come back as "parsed" or as an error code with a message; nothing may crash, hang or read past a buffer
(a run of either loop with 200,000 mutations, deep nesting and million-byte tokens was made while writing this test)."""
import ctypes
import json
import random
import re
import struct

from berth_b200 import _lib

from tests import test_config


def _mutate(rng, base: bytes, numbers=None) -> bytes:
    b = bytearray(base)
    for _ in range(rng.randint(1, 5)):
        if not b:
            break
        op = rng.randint(0, 4 if numbers else 3)
        if op == 0:
            b[rng.randrange(len(b))] = rng.randrange(256)
        elif op == 1:
            del b[rng.randrange(len(b))]
        elif op == 2:
            b.insert(rng.randrange(len(b) + 1), rng.choice(b'{}[]",:\\-+eE.0123456789tfn \x00\xff'))
        elif op == 3:
            b = b[:rng.randrange(len(b) + 1)]
        else:
            s = b.decode("latin1")
            found = list(re.finditer(r"\d+", s))
            if found:
                m = rng.choice(found)
                s = s[:m.start()] + rng.choice(numbers) + s[m.end():]
                b = bytearray(s.encode("latin1"))
    return bytes(b)


def test_config_parser_survives_mutations():
    lib = _lib.lib()
    value = test_config.sample()
    value["nested"] = {"a": [1, 2, {"b": "cé\n"}], "n": None, "t": True, "x": -1.5e-3}
    base = json.dumps(value).encode()
    rng = random.Random(1234)
    parsed = rejected = 0
    inputs = [base] + [_mutate(rng, base) for _ in range(4000)] + [b"[" * 100000, b'{"a":' * 50000, b'"' + b"\\" * 100001,
                                                                   b"1" * 1000000, b""]
    for buf in inputs:
        out = ctypes.c_void_p()
        rc = lib.berth_config_parse(buf, len(buf), ctypes.byref(out))
        if rc == 0:
            parsed += 1
            lib.berth_config_free(out)
        else:
            rejected += 1
            assert lib.berth_ckpt_last_error()
    assert parsed >= 1 and rejected >= 1000


def test_safetensors_header_reader_survives_mutations(tmp_path):
    lib = _lib.lib()
    header = {"__metadata__": {"format": "pt"},
              "model.layers.0.mlp.gate_proj.trellis": {"dtype": "I16", "shape": [8, 8, 64], "data_offsets": [0, 8192]},
              "model.layers.0.mlp.gate_proj.suh": {"dtype": "F16", "shape": [128], "data_offsets": [8192, 8448]},
              "model.layers.0.mlp.gate_proj.svh": {"dtype": "F16", "shape": [128], "data_offsets": [8448, 8704]},
              "model.norm.weight": {"dtype": "BF16", "shape": [128], "data_offsets": [8704, 8960]}}
    base = json.dumps(header).encode()
    data = bytes(8960)
    path = tmp_path / "model.safetensors"
    numbers = ["-1", "0", "18446744073709551615", "9223372036854775808", "99999999999999999999999", "8961", "1e9", "3.5"]
    rng = random.Random(99)
    cases = [(base, data, None)] + [(_mutate(rng, base, numbers), data, None) for _ in range(1500)]
    cases += [(base, data, n) for n in (0, 1, 7, len(base) + 1, len(base) + 10 ** 6, 2 ** 63, 2 ** 64 - 1)]   # the length word lies
    cases += [(base, b"", None), (b"{" * 200000, data, None)]
    opened = rejected = 0
    for hdr, dat, n in cases:
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(hdr) if n is None else n))
            f.write(hdr)
            f.write(dat)
        out = ctypes.c_void_p()
        rc = lib.berth_ckpt_open(str(tmp_path).encode(), ctypes.byref(out))
        if rc == 0:
            opened += 1
            assert lib.berth_ckpt_n_tensors(out) >= 0
            lib.berth_ckpt_close(out)
        else:
            rejected += 1
            assert lib.berth_ckpt_last_error()
    assert opened >= 1 and rejected >= 500
