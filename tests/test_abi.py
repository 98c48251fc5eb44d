"""The C-ABI library loads and exports every symbol the public header declares.
No compute is done here (no GPU needed)."""
import ctypes
import re

import pytest


def _declared_functions(header_text):
    text = re.sub(r"/\*.*?\*/", "", header_text, flags=re.S)
    return sorted(set(re.findall(r"\b(gptoss_moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    lib = pkg.load_library()
    names = _declared_functions(pkg.HEADER_PATH.read_text())
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_decode_header_symbols_are_exported(pkg):
    lib = pkg.load_library()
    text = (pkg.HEADER_PATH.parent / "gptoss_decode_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(gptoss_decode_[a-z0-9_]+)\s*\(", text)))
    assert len(names) >= 8
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    # the model config mirrors the 15 four-byte fields of the checkpoint header
    assert ctypes.sizeof(pkg.ModelConfig) == 60
    body = text[text.index("typedef struct {"):text.index("} gptoss_model_config_t;")]
    order = re.findall(r"\b(?:int|float)\s+([a-z_]+);", body)
    assert order == [f[0] for f in pkg.ModelConfig._fields_]


def test_version_string(pkg):
    assert b"sm_100a" in pkg.load_library().gptoss_moe_version()


def test_config_struct_matches_header(pkg):
    # 11 four-byte fields, no padding
    assert ctypes.sizeof(pkg.MoeConfig) == 44
    fields = [f[0] for f in pkg.MoeConfig._fields_]
    text = pkg.HEADER_PATH.read_text()
    body = text[text.index("typedef struct {"):text.index("} gptoss_moe_config_t;")]
    order = [m for m in re.findall(r"\b(?:int|float)\s+([a-z_]+);", body)]
    assert order == fields


def test_invalid_config_is_rejected_before_touching_cuda(pkg):
    with pytest.raises(pkg.MoeError) as ei:
        pkg.MoeEngine(100, 128, 8, 4)  # hidden_dim not a multiple of 8
    assert ei.value.code == pkg.GPTOSS_E_INVALID
    with pytest.raises(pkg.MoeError) as ei:
        pkg.MoeEngine(128, 128, 8, 9)  # top-k larger than supported
    assert ei.value.code == pkg.GPTOSS_E_INVALID
    with pytest.raises(pkg.MoeError) as ei:
        pkg.MoeEngine(128, 128, 6, 4, ep_rank=0, ep_size=4)  # experts not divisible
    assert ei.value.code == pkg.GPTOSS_E_INVALID


def test_no_cpu_fallback_without_gpu(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.MoeError) as ei:
        pkg.MoeEngine(128, 128, 8, 4)
    assert ei.value.code == pkg.GPTOSS_E_CUDA


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        pkg.load_library()


def test_getp_host_program_fails_loudly_without_gpu(pkg, tmp_path):
    """The C++ entry points build, link against the C ABI and refuse to run on a box
    without an sm_100 GPU (no fallback)."""
    import subprocess

    import torch

    from gpt_oss_b200 import build as native_build
    from gpt_oss_b200 import synth

    native_build.build_host()
    assert native_build.HOST_LIB.exists() and native_build.HARNESS.exists()
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    cfg = dict(synth.MINI_MODEL, vocab_size=64, n_layers=1)
    synth.write_model_bin(tmp_path / "m.bin", cfg, 1)
    (tmp_path / "req.txt").write_text("1\n1 2 3\n")
    res = subprocess.run([str(native_build.HARNESS), str(tmp_path / "m.bin"),
                          str(tmp_path / "req.txt"), str(tmp_path / "out.txt")],
                         capture_output=True, text=True, timeout=120)
    assert res.returncode != 0
    assert "no sm_100 GPU" in res.stderr
