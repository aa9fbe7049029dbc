"""Checkpoint files: the v1 text and v2 binary formats of src/engine/model/checkpoint.rs, written and
read by the library's host code (no GPU).  The cases follow the reference's own tests (:459-540:
round trip, legacy file without header, unknown comment lines, byte-stable re-save) and add the
failure messages of :89-160 and an independent reading of the binary form with Python's zlib."""
import struct
import zlib

import numpy as np
import pytest

from volta_b200 import VoltaB200Error
from volta_b200.checkpoint import BINARY_V2, TEXT_V1, Checkpoint


def sample():
    ck = Checkpoint()
    ck.add("w", np.array([[1.0, 2.0]], np.float32))
    ck.add("b", np.array([[0.25]], np.float32))
    return ck


def test_v1_roundtrip_preserves_parameters(tmp_path):
    p = tmp_path / "a.txt"
    sample().save(p)
    text = p.read_text()
    assert text.startswith("#volta-checkpoint:v1\n")
    assert text.splitlines()[2:] == ["b|1,1|0.25", "w|1,2|1,2"]        # sorted by name, no trailing newline
    assert not text.endswith("\n")
    got = Checkpoint.load(p).tensors()
    assert set(got) == {"w", "b"} and got["w"].shape == (1, 2) and got["b"].shape == (1, 1)
    assert np.array_equal(got["w"], [[1.0, 2.0]]) and np.array_equal(got["b"], [[0.25]])


def test_loader_accepts_the_reference_writers_output_and_legacy_files(tmp_path):
    p = tmp_path / "ref.txt"
    # what save_checkpoint writes (:19-40): nine decimals, "#writer:train_api"
    p.write_text("#volta-checkpoint:v1\n#writer:train_api\nb|1,1|0.250000000\nw|1,2|1.000000000,2.000000000")
    got = Checkpoint.load(p).tensors()
    assert np.array_equal(got["w"], [[1.0, 2.0]]) and np.array_equal(got["b"], [[0.25]])
    p.write_text("w|1,2|1.000000000,2.000000000\n")                     # legacy: no header at all
    got = Checkpoint.load(p).tensors()
    assert list(got) == ["w"] and got["w"].shape == (1, 2)
    p.write_text("\n\n#volta-checkpoint:v1\n#this-is-an-unknown-comment\n#another-comment=value\n\nw|1,2|1,2\n")
    assert Checkpoint.load(p).tensors()["w"].shape == (1, 2)
    p.write_text("s||3.5\nempty|0|\n")                                   # scalar (empty shape) and empty tensor
    got = Checkpoint.load(p).tensors()
    assert got["s"].shape == () and float(got["s"]) == 3.5 and got["empty"].shape == (0,)


def test_resave_is_byte_identical(tmp_path):
    a, b = tmp_path / "a.txt", tmp_path / "b.txt"
    sample().save(a)
    Checkpoint.load(a).save(b)
    assert a.read_bytes() == b.read_bytes()
    a2, b2 = tmp_path / "a.bin", tmp_path / "b.bin"
    sample().save(a2, BINARY_V2)
    Checkpoint.load(a2).save(b2, BINARY_V2)
    assert a2.read_bytes() == b2.read_bytes()


@pytest.mark.parametrize("content,message", [
    ("#volta-checkpoint:v9\nw|1|1", "Unsupported checkpoint version 'v9' at line 1"),
    ("#volta-checkpoint:v1\nw|1|1\n#volta-checkpoint:v2", "Unsupported checkpoint version 'v2' at line 3"),
    ("w|1,2", "Invalid checkpoint format at line 1"),
    ("#volta-checkpoint:v1\nw|1|2|3", "Invalid checkpoint format at line 2"),
    ("w|1,x|1,2", "Invalid shape dimension 'x' at line 1"),
    ("w|-1|1", "Invalid shape dimension '-1' at line 1"),
    ("w|2|1,abc", "Invalid data value 'abc' at line 1"),
    ("w|2|1,,2", "Invalid data value '' at line 1"),
    ("w|3|1,2", "Invalid tensor in checkpoint at line 1"),
])
def test_malformed_text_is_refused_with_the_reference_messages(tmp_path, content, message):
    p = tmp_path / "bad.txt"
    p.write_text(content)
    with pytest.raises(VoltaB200Error, match=message.replace("|", r"\|")):
        Checkpoint.load(p)


def test_missing_file_and_unwritable_names(tmp_path):
    with pytest.raises(VoltaB200Error, match="Failed to read checkpoint"):
        Checkpoint.load(tmp_path / "nope.txt")
    ck = Checkpoint()
    ck.add("a|b", np.zeros(1, np.float32))
    with pytest.raises(VoltaB200Error, match="cannot be written"):
        ck.save(tmp_path / "x.txt")
    with pytest.raises(VoltaB200Error, match="unknown checkpoint format"):
        sample().save(tmp_path / "y.txt", 4)


def hard_values():
    rs = np.random.RandomState(5)
    v = np.concatenate([
        rs.randn(4000).astype(np.float32), (rs.randn(2000) * 1e-12).astype(np.float32),
        (rs.randn(2000) * 1e20).astype(np.float32),
        np.array([0.0, -0.0, 1e-45, -1e-45, 1.17549435e-38, 3.4028235e38, -3.4028235e38, 1 / 3, 16777217.0], np.float32),
    ])
    return v


@pytest.mark.parametrize("fmt", [TEXT_V1, BINARY_V2])
def test_every_float_survives_bit_for_bit(tmp_path, fmt):
    v = hard_values()
    ck = Checkpoint()
    ck.add("layer0.weight", v[:8000].reshape(80, 100))
    ck.add("layer0.bias", v[8000:])
    p = tmp_path / "c"
    ck.save(p, fmt)
    got = Checkpoint.load(p).tensors()
    assert got["layer0.weight"].shape == (80, 100)
    assert np.array_equal(got["layer0.weight"].view(np.uint32).ravel(), v[:8000].view(np.uint32))
    assert np.array_equal(got["layer0.bias"].view(np.uint32), v[8000:].view(np.uint32))


def parse_v2_payload(payload):
    (count,), pos, out = struct.unpack_from("<I", payload, 0), 4, {}
    for _ in range(count):
        (nl,) = struct.unpack_from("<H", payload, pos); pos += 2
        name = payload[pos:pos + nl].decode(); pos += nl
        (ndim,) = struct.unpack_from("<I", payload, pos); pos += 4
        dims = struct.unpack_from("<%dI" % ndim, payload, pos); pos += 4 * ndim
        (ne,) = struct.unpack_from("<I", payload, pos); pos += 4
        out[name] = np.frombuffer(payload, "<f4", ne, pos).reshape(dims); pos += 4 * ne
    assert pos == len(payload)
    return out


def test_binary_layout_read_independently(tmp_path):
    """magic, then a zlib stream (stored blocks of at most 65535 bytes, Adler-32 trailer) that any
    inflater reads; payload as :162-198."""
    v = hard_values()                       # 40 KB: with the second tensor the payload spans two blocks
    ck = Checkpoint()
    ck.add("zeta", v.reshape(1, -1))
    ck.add("alpha", np.arange(12000, dtype=np.float32).reshape(3, 40, 100))
    p = tmp_path / "c.bin"
    ck.save(p, BINARY_V2)
    raw = p.read_bytes()
    assert raw[:8] == b"VOLTA\x02\x00\x00" and raw[8:10] == b"\x78\x9c"
    payload = zlib.decompress(raw[8:])      # checks block framing and the Adler-32
    assert len(payload) > 65535 and len(raw) == 8 + 2 + len(payload) + 5 * ((len(payload) + 65534) // 65535) + 4
    got = parse_v2_payload(payload)
    assert list(got) == ["alpha", "zeta"]   # sorted by name
    assert got["alpha"].shape == (3, 40, 100) and np.array_equal(got["zeta"].view(np.uint32).ravel(), v.view(np.uint32))


def test_binary_written_elsewhere_loads_and_real_deflate_is_refused(tmp_path):
    body = struct.pack("<I", 1) + struct.pack("<H", 1) + b"w" + struct.pack("<III", 2, 1, 2) + struct.pack("<I", 2) + \
        np.array([1.0, 2.0], "<f4").tobytes()
    stored = zlib.compressobj(level=0)
    p = tmp_path / "ext.bin"
    good = b"VOLTA\x02\x00\x00" + stored.compress(body) + stored.flush()
    p.write_bytes(good)
    got = Checkpoint.load(p).tensors()
    assert got["w"].shape == (1, 2) and np.array_equal(got["w"], [[1.0, 2.0]])
    p.write_bytes(b"VOLTA\x02\x00\x00" + zlib.compress(body * 50, 6))
    with pytest.raises(VoltaB200Error, match="BTYPE=[12] not supported"):     # as the reference's inflater (:367-373)
        Checkpoint.load(p)
    p.write_bytes(good[:8 + 9])                                               # cut inside the first block
    with pytest.raises(VoltaB200Error):
        Checkpoint.load(p)


def test_fixed_nine_decimals_are_the_reference_writers_bytes(tmp_path):
    """Format 3 prints `{v:.9}` as save_checkpoint does (checkpoint.rs:35), so a file of ours and a file of
    Volta's with the same tensors are the same bytes but for the writer line; small values then lose bits,
    which is why nine significant digits stay the default."""
    ck = Checkpoint()
    ck.add("fc1.weight", np.array([[1.0, -2.5, 1.2345678e-7]], np.float32))
    ck.add("fc1.bias", np.array([0.25], np.float32))
    p = tmp_path / "f.txt"
    ck.save(p, 3)
    assert p.read_text().splitlines()[2:] == ["fc1.bias|1|0.250000000", "fc1.weight|1,3|1.000000000,-2.500000000,0.000000123"]
    back = Checkpoint.load(p).tensors()
    assert back["fc1.weight"][0, 2] == np.float32(0.000000123)         # lossy, as in the reference
    ck.save(p, TEXT_V1)
    assert np.array_equal(Checkpoint.load(p).tensors()["fc1.weight"].view(np.uint32),
                          np.array([[1.0, -2.5, 1.2345678e-7]], np.float32).view(np.uint32))


@pytest.mark.parametrize("token", ["0x1p3", " 1.0", "1.0 ", "1_000", "1e", ".", "", "+-1", "1.0f"])
def test_reader_takes_only_what_rust_parses_as_f32(tmp_path, token):
    """The reference parses every value with f32::from_str (checkpoint.rs:141): no hexadecimal floats,
    no blanks inside a value.  A file accepted here must also load in Volta."""
    p = tmp_path / "bad.txt"
    p.write_text("#volta-checkpoint:v1\nw|3|1.0,%s,2.0" % token)   # in the middle: line ends are trimmed, as in the reference
    with pytest.raises(VoltaB200Error, match="Invalid data value|Invalid tensor"):
        Checkpoint.load(p)


@pytest.mark.parametrize("token,value", [("1.", 1.0), (".5", 0.5), ("+2", 2.0), ("-1e-3", -1e-3), ("3E2", 300.0),
                                         ("inf", np.inf), ("-Infinity", -np.inf)])
def test_reader_accepts_rusts_other_spellings(tmp_path, token, value):
    p = tmp_path / "ok.txt"
    p.write_text("w|1|%s" % token)
    assert Checkpoint.load(p).tensors()["w"][0] == np.float32(value)
    p.write_text("w|1|NaN")
    assert np.isnan(Checkpoint.load(p).tensors()["w"][0])


def _match(layers, ck, names=None):
    import ctypes as C
    from volta_b200 import load_library
    from volta_b200.lib import Config
    lib = load_library()
    cfg = Config()
    cfg.n_sizes = len(layers)
    for i, v in enumerate(layers):
        cfg.layers[i] = v
    cfg.batch = 4
    arr, n = (None, 0) if names is None else ((C.c_char_p * len(names))(*[None if v is None else v.encode() for v in names]), len(names))
    rc = lib.volta_b200_checkpoint_match(C.byref(cfg), ck.h, arr, n)
    return rc, lib.volta_b200_last_error(None).decode()


def test_layer_names_of_a_volta_model_are_found(tmp_path):
    """Volta names tensors after the layers ("{name}.weight", "{name}.bias", model/layers.rs:52-58).  A file
    written the way its save_checkpoint writes one (sorted by name, nine decimals) resolves onto a 3-4-2
    topology without the caller naming the layers, and with explicit names in any order."""
    p = tmp_path / "volta.txt"
    w1, w2 = np.arange(12, dtype=np.float32).reshape(3, 4), np.arange(8, dtype=np.float32).reshape(4, 2)
    rows = {"fc1.weight": w1, "fc1.bias": np.zeros(4, np.float32), "fc2.weight": w2, "fc2.bias": np.ones(2, np.float32)}
    lines = ["#volta-checkpoint:v1", "#writer:train_api"]
    for name in sorted(rows):
        t = rows[name]
        lines.append("%s|%s|%s" % (name, ",".join(map(str, t.shape)), ",".join("%.9f" % v for v in t.ravel())))
    p.write_text("\n".join(lines))
    ck = Checkpoint.load(p)
    assert _match([3, 4, 2], ck)[0] == 4                                  # two weights + two biases
    assert _match([3, 4, 2], ck, ["fc1", "fc2"])[0] == 4
    rc, why = _match([3, 4, 2], ck, ["fc2", "fc1"])
    assert rc == -1 and "wrong shape" in why
    rc, why = _match([3, 4, 2], ck, ["encoder", "head"])
    assert rc == -1 and "no '<name>.weight'" in why
    rc, why = _match([3, 4, 4, 2], ck)                                    # three layers, two pairs in the file
    assert rc == -1 and "pass the layer names" in why
    rc, why = _match([3, 5, 2], ck)
    assert rc == -1 and "wrong shape" in why


def test_a_checkpoint_without_any_known_parameter_is_refused():
    ck = Checkpoint()
    ck.add("something.else", np.zeros(3, np.float32))
    rc, why = _match([3, 4, 2], ck)
    assert rc == -1 and why
    own = Checkpoint()
    own.add("layer1.bias", np.zeros(2, np.float32))                       # a partial file of this library's names
    assert _match([3, 4, 2], own)[0] == 1
