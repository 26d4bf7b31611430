"""There is one product path: the compiled sm_100a kernels on a CUDA device.  Without them the library says so;
it does not fall back to anything."""

import pytest

from starter_b200.csrc import build
from starter_b200.csrc.build import BuildError


def test_a_session_on_the_cpu_needs_a_call_table_of_its_own(tiny_folders):
    from starter_b200.engine.session import Session
    with pytest.raises(ValueError, match="CUDA device"):
        Session(tiny_folders["A"], dtype="float32", device="cpu")


def test_no_device_is_an_error(monkeypatch):
    import torch
    import starter_b200.csrc.ops as ops
    monkeypatch.setattr(ops, "_OPS", None)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(BuildError, match="no CUDA device"):
        ops.get_ops(verbose=False)


def test_a_missing_compiler_is_an_error_that_names_where_it_looked(monkeypatch, tmp_path):
    monkeypatch.setattr(build, "_LIB", None)
    monkeypatch.setenv("STARTER_B200_BUILD_DIR", str(tmp_path))      # nothing built there
    monkeypatch.setenv("PATH", str(tmp_path))
    monkeypatch.delenv("CUDA_HOME", raising=False)
    monkeypatch.delenv("CUDA_PATH", raising=False)
    monkeypatch.setattr(build.Path, "is_file", lambda self: False if self.name == "nvcc" else build.Path.exists(self))
    with pytest.raises(BuildError, match="nvcc was not found"):
        build.load(verbose=False)


def test_a_source_that_does_not_compile_is_an_error_with_the_compiler_s_words(monkeypatch, tmp_path):
    bad = tmp_path / "src"
    bad.mkdir()
    (bad / "broken.cu").write_text("this is not CUDA\n")
    monkeypatch.setattr(build, "_LIB", None)
    monkeypatch.setattr(build, "HERE", bad)
    monkeypatch.setenv("STARTER_B200_BUILD_DIR", str(tmp_path / "out"))
    with pytest.raises(BuildError, match="nvcc failed on broken.cu"):
        build.load(verbose=False)
