"""B200-native render hot path of MLP Splatting.

Public surface (mirrors the reference's scannet package for this path):
  cumodel.NeuralPrimitiveSceneTileCUDA   scannet/cumodel.py:655
  camera.ray_cone_candidates             scannet/camera.py:102-146
  primitive_csr.group_records / PrimitiveCSR   scannet/primitive_csr.py:14-29
  primitive_gemm.GroupLayout / prepare_groups / resolve_groups / grouped_forward   scannet/primitive_gemm.py
  engine.PackedScene / FrameRenderer     device-resident scene + per-frame driver over the C ABI
  synthetic                              seeded scenes and cameras
Importing the package does not need a GPU; rendering does, and raises when libmlpsp_b200.so is absent.
"""
from . import synthetic  # noqa: F401

__all__ = ["synthetic", "engine", "cumodel", "camera", "primitive_csr", "primitive_gemm", "sharding"]


def __getattr__(name):
    if name in ("engine", "cumodel", "camera", "primitive_csr", "primitive_gemm", "sharding", "_lib"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
