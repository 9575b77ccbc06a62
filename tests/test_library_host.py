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


def test_layer_entries_reject_bad_arguments(lib):
  """The entries of the KPConv / PointConv / pooling layers check their scalar
  arguments before any launch."""
  i64, f = ctypes.c_int64, ctypes.c_float
  rc = lib.tfgpc_kp_basis(None, 3, 16, 17, i64(4), None, None, None, None, f(1.0), f(1.0), 0, None)
  assert rc == 1 and b"kernel points" in lib.tfgpc_last_error()
  rc = lib.tfgpc_kp_basis(None, 3, 16, 15, i64(4), None, None, None, None, f(1.0), f(1.0), 2, None)
  assert rc == 1 and b"interpolation" in lib.tfgpc_last_error()
  rc = lib.tfgpc_kp_basis(None, 3, 12, 5, i64(4), None, None, None, None, f(1.0), f(1.0), 0, None)
  assert rc == 1 and b"basis functions" in lib.tfgpc_last_error()
  rc = lib.tfgpc_neighborhood_pool(None, 2, 8, i64(4), i64(4), i64(4), None, None, None, None)
  assert rc == 1 and b"mode" in lib.tfgpc_last_error()
  rc = lib.tfgpc_global_pool(None, 0, 8, i64(4), i64(0), None, None, None, None,
                             ctypes.c_size_t(0))
  assert rc == 1 and b"batch size" in lib.tfgpc_last_error()
  rc = lib.tfgpc_scale_bias_activation(None, i64(4), 8, None, f(1.0), None, 3, f(0.0))
  assert rc == 1 and b"activation" in lib.tfgpc_last_error()
  rc = lib.tfgpc_mcconv_workspace_bytes(16, 128, 256, i64(100), i64(100), 1)
  assert rc > 0
  assert lib.tfgpc_global_pool_workspace_bytes(i64(32)) >= 128
