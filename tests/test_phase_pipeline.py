"""Host-side tests of the phase-aware dispatch surface (no GPU): the reference's phase
heuristic (src/inference/phase_pipeline.mm:42-51), per-phase configurations, and the decode /
tensor-core threshold option with its environment override."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_detect_phase_follows_the_reference_heuristic():
    from metal_native.phase_pipeline import InferencePhase, detect_phase
    D, P = InferencePhase.Decode, InferencePhase.Prefill
    cases = {(1, 1): D, (8, 1): D, (64, 1): D, (1, 2): D, (1, 4): D, (1, 5): P, (2, 2): P, (2, 4): P, (1, 512): P,
             (16, 128): P}
    for (batch, seq), want in cases.items():
        assert detect_phase(batch, seq) is want, (batch, seq)


def test_configurations_and_fallback():
    from metal_native.phase_pipeline import InferencePhase, PhaseConfig, PhasePipeline

    class Fake:
        def __init__(self):
            self.opts = {"gemv_max_m": 0}

        def set_option(self, k, v):
            self.opts[k] = v

    be = Fake()
    p = PhasePipeline(backend=be)
    assert p.current_phase() is InferencePhase.Unknown
    assert p.active_config() == p.prefill_config()            # Unknown falls back to prefill
    assert p.decode_config().matmul_strategy == "gemv" and p.prefill_config().matmul_strategy == "gemm"
    assert p.prefill_config().gemv_max_m == 0                 # threshold left to the library
    assert [p.strategy_for(m) for m in (16, 17, 64, 65)] == ["gemv", "auto", "auto", "gemm"]
    p.set_decode_config(PhaseConfig("gemv", 16, True))
    p.set_prefill_config(PhaseConfig("gemm", 8, False))
    p.set_phase(InferencePhase.Decode)
    assert p.apply().gemv_max_m == 16 and be.opts["gemv_max_m"] == 16
    assert p.strategy_for(16) == "gemv" and p.strategy_for(17) == "gemm"
    p.auto_detect_phase(4, 128)
    assert p.apply().gemv_max_m == 8 and be.opts["gemv_max_m"] == 8
    cfg = p.prefill_config()
    cfg.gemv_max_m = 1                                        # a copy: the pipeline's own is untouched
    assert p.prefill_config().gemv_max_m == 8
    with pytest.raises(ValueError):
        p.set_decode_config(PhaseConfig("vecmat", 8))
    with pytest.raises(ValueError):
        p.set_decode_config(PhaseConfig("gemv", 64))
    step = object()
    assert p.capture_step(step) is step                      # prefill: no capture, the step itself


def test_threshold_option_and_environment_override():
    code = ("import sys; sys.path.insert(0, r'%s'); from metal_native import _C; "
            "print(_C.get_option('gemv_max_m'), _C.select_path(12, 4096, 4096, 128, 'int4'), "
            "_C.select_path(4, 4096, 4096, 128, 'int4'), _C.select_path(33, 4096, 4096, 128, 'int4'), "
            "_C.select_path(28, 4096, 4096, 4096, 'int8'))" % (ROOT / "metal-native_b200"))
    for env_val, want in ((None, "0 gemv gemv gemm gemm"), ("0", "0 gemv gemv gemm gemm"), ("8", "8 gemm gemv gemm gemm"),
                          ("32", "32 gemv gemv gemm gemv"), ("99", "0 gemv gemv gemm gemm"), ("x", "0 gemv gemv gemm gemm")):
        env = dict(os.environ)
        env.pop("METAL_NATIVE_GEMV_MAX_M", None)
        if env_val is not None:
            env["METAL_NATIVE_GEMV_MAX_M"] = env_val
        r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        assert r.stdout.strip() == want, (env_val, r.stdout)


def test_options_validate_and_round_trip():
    from metal_native import _C
    assert _C.get_option("weights_immutable") == 0
    _C.set_option("weights_immutable", 1)
    assert _C.get_option("weights_immutable") == 1
    _C.set_option("weights_immutable", 0)
    for name, bad in (("weights_immutable", 2), ("peer_wait_polls", 0), ("gemv_max_m", -1), ("gemv_max_m", 33)):
        with pytest.raises(_C.MetalNativeError, match="InvalidArgument"):
            _C.set_option(name, bad)
    with pytest.raises(_C.MetalNativeError):
        _C.set_option("nope", 1)
    assert _C._lib.mnq_get_option(77) == -1
    # the threshold left to the library: by weight format and activation type
    import torch
    sp = _C.select_path
    assert _C.get_option("gemv_max_m") == 0
    assert [sp(m, 4096, 4096, 4096, "int8", torch.bfloat16) for m in (16, 17)] == ["gemv", "gemm"]
    assert [sp(m, 16384, 4096, 128, "int8", torch.float16) for m in (32, 33)] == ["gemv", "gemm"]
    assert [sp(m, 16384, 4096, 128, "int4", torch.float16) for m in (32, 33)] == ["gemv", "gemm"]
    # small layers of few rows (fewer than 8192, less than 24 MB): the tensor-core kernel from 17 tokens
    assert [sp(m, 4096, 4096, 128, "int4", torch.float16) for m in (16, 17)] == ["gemv", "gemm"]
    assert [sp(m, 4096, 4096, 128, "int8", torch.float16) for m in (16, 17)] == ["gemv", "gemm"]
    assert [sp(m, 4096, 14336, 128, "int4", torch.float16) for m in (32, 33)] == ["gemv", "gemm"]   # 29 MB
    assert [sp(m, 4096, 4096, 128, "int4", torch.bfloat16) for m in (32, 33, 64, 65)] == ["gemv", "gemv", "gemv", "gemm"]
    assert [sp(m, 4096, 4096, 4096, "int4", torch.bfloat16) for m in (32, 33)] == ["gemv", "gemm"]   # one scale per row, no zeros: integer tiles
    # fp16 activations with bf16 scales above the decode threshold: the any-shape kernel, and it says so
    assert _C.select_path(64, 4096, 4096, 128, "int4", torch.float16, scale_dtype=torch.bfloat16) == "generic"
    assert _C.select_path(64, 4096, 4096, 128, "int4", torch.float16, scale_dtype=torch.float16) == "gemm"
    assert _C.select_path(65, 4096, 4096, 128, "int4", torch.bfloat16, scale_dtype=torch.float16) == "gemm"
