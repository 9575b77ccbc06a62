"""ctypes binding of libtfgpc.so, the C ABI declared in include/tfgpc.h.

There is no fallback: if the library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtfgpc.so")

_lib = None

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_vp = ctypes.c_void_p
c_sz = ctypes.c_size_t


class TfgpcError(RuntimeError):
  """A C-ABI call returned a non-zero status."""

  def __init__(self, code, message):
    super().__init__("tfgpc error %d: %s" % (code, message))
    self.code = code


# Every symbol include/tfgpc.h declares, with its return type.
SYMBOLS = {
    "tfgpc_last_error": ctypes.c_char_p,
    "tfgpc_version": c_int,
    "tfgpc_compute_keys": c_int,
    "tfgpc_compute_aabb": c_int,
    "tfgpc_compute_pdf_at_samples": c_int,
    "tfgpc_sort_keys_workspace_bytes": c_sz,
    "tfgpc_sort_keys_desc": c_int,
    "tfgpc_build_grid_ds": c_int,
    "tfgpc_find_neighbors_workspace_bytes": c_sz,
    "tfgpc_find_neighbors_count": c_int,
    "tfgpc_find_neighbors_fill": c_int,
    "tfgpc_find_neighbors_count_ordered": c_int,
    "tfgpc_find_neighbors_fill_ordered": c_int,
    "tfgpc_grid_neighborhood_workspace_bytes": c_sz,
    "tfgpc_grid_neighborhood_ds_elems": c_sz,
    "tfgpc_grid_neighborhood_count": c_int,
    "tfgpc_grid_cells": c_int,
    "tfgpc_pack_points_density": c_int,
    "tfgpc_find_neighbors_fill_fused": c_int,
    "tfgpc_original_neighbor_ids": c_int,
    "tfgpc_find_neighbors_static_max_samples": c_i64,
    "tfgpc_find_neighbors_count_static": c_int,
    "tfgpc_compute_pdf": c_int,
    "tfgpc_compute_pdf_pt_grads": c_int,
    "tfgpc_basis_proj": c_int,
    "tfgpc_basis_proj_grads": c_int,
    "tfgpc_basis_proj_workspace_bytes": c_sz,
    "tfgpc_basis_proj_ws": c_int,
    "tfgpc_basis_proj_grads_ws": c_int,
    "tfgpc_sampling_workspace_bytes": c_sz,
    "tfgpc_sampling_count": c_int,
    "tfgpc_sampling_count_symmetric": c_int,
    "tfgpc_sampling_store": c_int,
    "tfgpc_mcconv_workspace_bytes": c_sz,
    "tfgpc_mcconv_forward": c_int,
    "tfgpc_mcconv_backward": c_int,
    "tfgpc_mcconv_status": c_int,
    "tfgpc_mcconv_grouped_supported": c_int,
    "tfgpc_mcconv_group_plan_bytes": c_sz,
    "tfgpc_mcconv_group_plan": c_int,
    "tfgpc_mcconv_forward_grouped": c_int,
    "tfgpc_mcconv_backward_grouped": c_int,
    "tfgpc_kernel_basis_split": c_int,
    "tfgpc_kernel_basis": c_int,
    "tfgpc_kernel_basis_grads": c_int,
    "tfgpc_kernel_mlp_basis": c_int,
    "tfgpc_kernel_mlp_grads": c_int,
    "tfgpc_kp_basis": c_int,
    "tfgpc_pointconv_pdf": c_int,
    "tfgpc_neighborhood_pool": c_int,
    "tfgpc_global_pool_workspace_bytes": c_sz,
    "tfgpc_global_pool": c_int,
    "tfgpc_add_bias": c_int,
    "tfgpc_scale_bias_activation": c_int,
    "tfgpc_matmul_workspace_bytes": c_sz,
    "tfgpc_matmul_f32": c_int,
    "tfgpc_debug_bounded_wait": c_int,
    "tfgpc_read_device": c_int,
    "tfgpc_profile_enable": c_int,
    "tfgpc_profile_collect": c_int,
}


def lib():
  """Loads the library once; raises if it has not been built."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise RuntimeError(
          "libtfgpc.so is missing (%s): build it with "
          "`python -m tensorflow_graphics_point_clouds_b200.build`; there is no "
          "CPU or eager fallback" % LIB_PATH)
    handle = ctypes.CDLL(LIB_PATH)
    for name, restype in SYMBOLS.items():
      getattr(handle, name).restype = restype
    _lib = handle
  return _lib


def check(code):
  if code != 0:
    raise TfgpcError(code, lib().tfgpc_last_error().decode())


def ptr(t):
  """Device (or host) address of a torch tensor as a void*; None -> NULL."""
  if t is None:
    return c_vp(0)
  return c_vp(t.data_ptr())


def profile_enable(on=True):
  """Turns the library's per-launch CUDA-event timing on or off (this thread)."""
  check(lib().tfgpc_profile_enable(c_int(int(on))))


def profile_collect(max_records=65536):
  """Returns [(name, milliseconds)] of every launch group since the last call."""
  names = ctypes.create_string_buffer(64 * max_records)
  ms = (ctypes.c_float * max_records)()
  count = c_int(0)
  check(lib().tfgpc_profile_collect(names, c_sz(len(names)), ms, c_int(max_records),
                                    ctypes.byref(count)))
  labels = names.value.decode().split("\n")[:count.value]
  return [(labels[i], float(ms[i])) for i in range(count.value)]
