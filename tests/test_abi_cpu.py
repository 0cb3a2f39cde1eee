"""The C-ABI library loads without a GPU and exports every symbol include/mlpsp.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mlpsp.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlpsp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mlp_splatting_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "build the library first: python mlp-splatting_b200/build.py"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mlpsp.h but not exported"
    assert set(_lib.EXPORTS) == set(names), "binding table and header disagree"


def test_struct_layout_and_pure_host_queries():
    from mlp_splatting_b200 import _lib
    lib = _lib.load()   # checks ABI version and struct sizes
    assert lib.mlpsp_frame_scratch_bytes(1000, 128, 96, 8, 10000, 50000) > 0
    assert lib.mlpsp_frame_scratch_bytes(-1, 128, 96, 8, 10000, 50000) == -1
    assert lib.mlpsp_group_records_scratch_bytes(1000, 10) > 0
    assert lib.mlpsp_mlp_grouped_scratch_bytes(1000, 10) > 0


def test_argument_errors_need_no_gpu():
    from mlp_splatting_b200 import _lib
    lib = _lib.load()
    assert lib.mlpsp_normalize_rows(None, None, 4, 5, None) == -1
    assert b"dim must be 3 or 4" in lib.mlpsp_last_error()
    sc, fr = _lib.Scene(), _lib.Frame()
    fr.width, fr.height, fr.tile, fr.threshold = 64, 48, 16, 0.5
    assert lib.mlpsp_render_frame(ctypes.byref(sc), ctypes.byref(fr), None) == -1
    assert b"8x8 tiles" in lib.mlpsp_last_error()


def test_null_segment_arrays_are_refused_before_any_launch():
    """mlpsp_grouped_weight_gradients with segments to process but no segment arrays: an argument error, found by the
    host-side checks (this machine has no GPU to launch on)."""
    from mlp_splatting_b200 import _lib
    lib = _lib.load()
    sc = _lib.Scene()
    sc.n, sc.hidden, sc.num_freq = 4, 32, 6
    fake = 0x1000     # never dereferenced: the call must stop at its argument checks
    sc.W1 = sc.b1 = sc.W2 = sc.b2 = sc.W3 = sc.freq = sc.att = fake
    rc = lib.mlpsp_grouped_weight_gradients(ctypes.byref(sc), fake, fake, fake, None, None, None, None, 3, 128, 0, 1.0,
                                            None, fake, fake, None)
    assert rc == -1 and b"null pointer" in lib.mlpsp_last_error()
    assert lib.mlpsp_records_reverse(None, None, None, None, None, None, None, None, 0, 0, 0, None, None, None, None, None) == -1


def test_batch_and_precision_arguments_are_checked_before_any_launch():
    """mlpsp_render_frames and the precision argument of mlpsp_grouped_weight_gradients: argument errors come from the
    host-side checks."""
    from mlp_splatting_b200 import _lib
    lib = _lib.load()
    sc = _lib.Scene()
    frames = (_lib.Frame * 2)()
    assert lib.mlpsp_render_frames(ctypes.byref(sc), frames, 0, None) == -1
    assert b"need 1..64 frames" in lib.mlpsp_last_error()
    assert lib.mlpsp_render_frames(ctypes.byref(sc), frames, 65, None) == -1
    frames[0].width, frames[0].height, frames[0].tile, frames[0].threshold = 64, 48, 16, 0.5
    assert lib.mlpsp_render_frames(ctypes.byref(sc), frames, 2, None) == -1
    assert b"8x8 tiles" in lib.mlpsp_last_error()
    sc.n, sc.hidden, sc.num_freq = 4, 32, 6
    fake = 0x1000
    sc.W1 = sc.b1 = sc.W2 = sc.b2 = sc.W3 = sc.freq = sc.att = fake
    rc = lib.mlpsp_grouped_weight_gradients(ctypes.byref(sc), fake, fake, fake, None, fake, fake, fake, 3, 128, 7, 1.0,
                                            fake, fake, fake, None)
    assert rc == -1 and b"unsupported operand precision 7" in lib.mlpsp_last_error()


def test_product_never_imports_oracle():
    pkg = os.path.join(ROOT, "mlp-splatting_b200")
    for dirpath, _d, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower().replace("# oracle", ""), f


def test_missing_library_fails_loudly(monkeypatch):
    from mlp_splatting_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libmlpsp_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_weight_gradient_safety_policy_on_a_fake_launch():
    """The host policy of grouped_weight_gradients (scannet/primitive_gemm.py:64-98) without a GPU: a finite result
    is returned as is, a non-finite mixed-precision result is recomputed once in unscaled FP32 with a warning, a
    non-finite FP32 result raises, and the counters follow."""
    import warnings

    import pytest
    import torch
    from mlp_splatting_b200 import primitive_gemm as pg
    pg.get_grouped_vjp_safety_stats(reset=True)
    calls = []

    def launch_ok(dtype, scale):
        calls.append((dtype, scale))
        return "result", False

    assert pg._checked_grouped_vjp(launch_ok, torch.float16, 4096.0) == "result"
    assert calls == [(torch.float16, 4096.0)]

    def launch_mixed_bad(dtype, scale):
        calls.append((dtype, scale))
        return ("fp32 result", False) if dtype == torch.float32 else ("garbage", True)

    calls.clear()
    with pytest.warns(RuntimeWarning, match="retrying with IEEE FP32"):
        assert pg._checked_grouped_vjp(launch_mixed_bad, torch.bfloat16, 1.0) == "fp32 result"
    assert calls == [(torch.bfloat16, 1.0), (torch.float32, 1.0)]

    def launch_bad(dtype, scale):
        return "garbage", True

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with pytest.raises(FloatingPointError, match="IEEE FP32 MLP VJP is nonfinite"):
            pg._checked_grouped_vjp(launch_bad, torch.float16, 4096.0)
        with pytest.raises(FloatingPointError):
            pg._checked_grouped_vjp(launch_bad, torch.float32, 1.0)
    stats = pg.get_grouped_vjp_safety_stats(reset=True)
    assert stats == {"calls": 4, "mixed_calls": 3, "fp32_fallbacks": 2, "fp32_nonfinite_failures": 2}
    assert pg.get_grouped_vjp_safety_stats()["calls"] == 0


def test_build_configuration_variables_select_run_time_arguments(monkeypatch):
    """The reference's build-time environment variables (scannet/cumodel.py:96-130), same checks and texts."""
    import pytest
    from mlp_splatting_b200.cumodel import _tile_ext_build_config
    for k in ("MLPSP_TILE_CANDIDATE_CAPACITY", "MLPSP_TRAINING_BACKEND", "MLPSP_CSR_MAX_HITS", "MLPSP_NVCC_MAXRREGCOUNT"):
        monkeypatch.delenv(k, raising=False)
    assert _tile_ext_build_config() == {"tile_candidate_capacity": 1536, "csr_max_hits": None, "tile_size": 8}
    monkeypatch.setenv("MLPSP_TILE_CANDIDATE_CAPACITY", "768")
    monkeypatch.setenv("MLPSP_NVCC_MAXRREGCOUNT", "64")
    assert _tile_ext_build_config()["tile_candidate_capacity"] == 768
    monkeypatch.setenv("MLPSP_TILE_CANDIDATE_CAPACITY", "1000")
    with pytest.raises(ValueError, match="MLPSP_TILE_CANDIDATE_CAPACITY must be 768 or 1536"):
        _tile_ext_build_config()
    monkeypatch.setenv("MLPSP_TILE_CANDIDATE_CAPACITY", "1536")
    monkeypatch.setenv("MLPSP_TRAINING_BACKEND", "csr")
    assert _tile_ext_build_config()["csr_max_hits"] == 128
    monkeypatch.setenv("MLPSP_CSR_MAX_HITS", "256")
    assert _tile_ext_build_config()["csr_max_hits"] == 256
    monkeypatch.setenv("MLPSP_CSR_MAX_HITS", "300")
    with pytest.raises(ValueError, match="MLPSP_CSR_MAX_HITS must be 128, 256 or 512"):
        _tile_ext_build_config()


def test_bench_combines_the_ranks_side_measurements():
    """bench.combine_other_workloads: the slowest rank sets the step time, record counts add up, a failure on any rank
    is reported in place of figures, and a record measured by rank 0 alone passes through."""
    import bench
    def rec(dev_ms, records, wt, ws, bits=0):
        return {"frames_per_sec": -1.0, "ms_per_step": -1.0, "steps": 2, "views_per_step": 32, "status_bits": bits,
                "local": {"dev_ms": dev_ms, "records": records, "work_total": wt, "work_small": ws}}
    out = bench.combine_other_workloads([{"a": rec(100.0, 1000.0, 10.0, 4.0), "b": rec(5.0, 1.0, 1.0, 0.0), "g": {"fp32_ms": 1.0}},
                                         {"a": rec(160.0, 3000.0, 30.0, 6.0, bits=8), "b": {"failed": "RuntimeError: boom"},
                                          "g": {"fp32_ms": 1.0}}])
    a = out["a"]
    assert a["ms_per_step"] == 80.0 and a["frames_per_sec"] == 32 * 2 / 0.160 and a["records_per_step"] == 4000.0
    assert a["rows_per_evaluator_block"] == 100.0 and a["status_bits"] == 8 and "local" not in a
    assert abs(a["fill_of_evaluator_blocks"] - 4000.0 / (128 * 30 + 32 * 10)) < 1e-12
    assert "rank 1: RuntimeError: boom" in out["b"]["failed"]
    assert out["g"] == {"fp32_ms": 1.0}
