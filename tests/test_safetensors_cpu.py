"""The C++ .safetensors reader (include/anygpu/io/safetensors_file.hpp) against a file written here byte by byte: header with a
__metadata__ object (with braces and escaped quotes inside a string), F32 / F16 / BF16 tensors, a 3-D shape. Host code only, no GPU."""
import json
import os
import struct
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "cpp"))


def to_bf16_bits(a):
    u = np.asarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)  # round to nearest even


def test_safetensors_reader_reads_f32_f16_bf16(tmp_path):
    import build as cpp_build
    exe = cpp_build.SFT_OUT if os.path.exists(cpp_build.SFT_OUT) else cpp_build.build_sft_dump()
    r = np.random.default_rng(0)
    tensors = {
        "model.layers.0.mamba.in_proj.weight": ("F32", r.standard_normal((24, 16)).astype(np.float32)),
        "model.layers.0.mamba.conv1d.weight": ("F16", r.standard_normal((12, 1, 4)).astype(np.float32)),
        "model.layers.0.mamba.A_log": ("BF16", r.uniform(0, 3, 7).astype(np.float32)),
        "model.layers.0.mamba.norm.weight": ("BF16", np.ones(16, np.float32)),
    }
    header, blob, want = {"__metadata__": {"format": "pt", "odd": 'a {brace} and a [bracket], "quoted"'}}, b"", {}
    for name, (dt, a) in tensors.items():
        if dt == "F32":
            raw, back = a.tobytes(), a
        elif dt == "F16":
            h = a.astype(np.float16)
            raw, back = h.tobytes(), h.astype(np.float32)
        else:
            bits = to_bf16_bits(a)
            raw, back = bits.tobytes(), (bits.astype(np.uint32) << 16).view(np.float32)
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
        want[name] = (dt, a.shape, float(back.astype(np.float64).sum()), float((back.astype(np.float64) ** 2).sum()))
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    path = tmp_path / "t.safetensors"
    path.write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    out = subprocess.run([exe, str(path)], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [l for l in out.stdout.splitlines() if "|" in l]
    assert len(lines) == len(tensors)
    for line in lines:
        left, right = line.split("|")
        name, dt, *shape = left.split()
        s, s2 = (float(v) for v in right.split())
        wdt, wshape, ws, ws2 = want[name]
        assert dt == wdt and tuple(int(v) for v in shape) == tuple(wshape)
        assert abs(s - ws) <= 1e-6 * max(1.0, abs(ws)) and abs(s2 - ws2) <= 1e-6 * max(1.0, ws2), (name, s, ws, s2, ws2)


def test_safetensors_reader_refuses_truncated_and_corrupt_files(tmp_path):
    """A header length larger than the file, a header cut short and data_offsets that point past the end of the file must end
    with an error message and exit status 1, not with an unbounded allocation or silently empty tensors."""
    import build as cpp_build
    exe = cpp_build.SFT_OUT if os.path.exists(cpp_build.SFT_OUT) else cpp_build.build_sft_dump()
    a = np.arange(8, dtype=np.float32)
    hj = json.dumps({"t": {"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}}).encode()
    good = struct.pack("<Q", len(hj)) + hj + a.tobytes()
    bad_offsets = json.dumps({"t": {"dtype": "F32", "shape": [8], "data_offsets": [0, 64]}}).encode()
    cases = {
        "huge_header": struct.pack("<Q", 1 << 60) + hj + a.tobytes(),
        "cut_in_header": good[:8 + len(hj) // 2],
        "offsets_past_end": struct.pack("<Q", len(bad_offsets)) + bad_offsets + a.tobytes(),
        "empty": b"",
    }
    path = tmp_path / "ok.safetensors"
    path.write_bytes(good)
    assert subprocess.run([exe, str(path)], capture_output=True, text=True, timeout=60).returncode == 0
    for name, blob in cases.items():
        path = tmp_path / (name + ".safetensors")
        path.write_bytes(blob)
        out = subprocess.run([exe, str(path)], capture_output=True, text=True, timeout=60)
        assert out.returncode == 1, (name, out.returncode, out.stdout[-200:], out.stderr[-200:])
