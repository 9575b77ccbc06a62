"""Host-side checks that need no GPU: the C-ABI library loads, exports every
symbol that include/tfgpc.h declares, and rejects bad arguments before it
touches the device."""
import ctypes
import os
import re

import pytest

from tensorflow_graphics_point_clouds_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
  build.build()
  return _lib.lib()


def declared_symbols():
  text = open(os.path.join(ROOT, "include", "tfgpc.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(tfgpc_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
  names = declared_symbols()
  assert len(names) >= 16
  for name in names:
    assert hasattr(lib, name), name
  assert set(names) == set(_lib.SYMBOLS), "ctypes table and header disagree"


def test_version_and_empty_error(lib):
  assert lib.tfgpc_version() >= 1


def test_no_torch_types_in_header():
  text = open(os.path.join(ROOT, "include", "tfgpc.h")).read()
  assert "torch" not in text and "at::" not in text


@pytest.mark.parametrize("d", [1, 7])
def test_invalid_dimension_is_rejected(lib, d):
  rc = lib.tfgpc_compute_keys(None, d, ctypes.c_int64(4), None, None, ctypes.c_int64(1), None,
                              None, None, None)
  assert rc == 1
  assert b"dimension" in lib.tfgpc_last_error()


def test_invalid_basis_and_features_are_rejected(lib):
  i64 = ctypes.c_int64
  rc = lib.tfgpc_basis_proj(None, 12, 8, i64(1), i64(1), i64(1), None, None, None, None, None)
  assert rc == 1 and b"basis functions" in lib.tfgpc_last_error()
  rc = lib.tfgpc_basis_proj(None, 16, 9, i64(1), i64(1), i64(1), None, None, None, None, None)
  assert rc == 1 and b"input features" in lib.tfgpc_last_error()


def test_workspace_queries_grow_with_size(lib):
  i64 = ctypes.c_int64
  assert lib.tfgpc_find_neighbors_workspace_bytes(i64(10)) > 0
  assert (lib.tfgpc_sampling_workspace_bytes(i64(1 << 20))
          > lib.tfgpc_sampling_workspace_bytes(i64(1 << 10)))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
  with pytest.raises(RuntimeError, match="no\\s+CPU or eager fallback"):
    _lib.lib()
