"""Phase-aware dispatch surface for the quantised operator.

Mirror, for this one path, of the reference's ``PhasePipeline``
(``include/metal_native/inference/phase_pipeline.h:23-127``,
``src/inference/phase_pipeline.mm:17-167``): it tells prefill from decode by batch size and
sequence length, keeps one configuration per phase and applies the active one.  What a
configuration can actually steer here is the operator's kernel choice: ``gemv_max_m`` is the
largest token count that takes the streaming decode kernels (the reference's fixed
``use_vecmat = M <= 8``, ``src/ops/matmul.mm:946``); larger problems run the tensor-core
kernel.  The reference's lazy-commit batching of a decode step
(``src/dispatch/command_pipeline.mm:124-137``) becomes CUDA-graph capture:
``capture_step`` records a step once and replays it with one launch.
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass, replace

MATMUL_STRATEGIES = ("gemv", "gemm", "auto")


class InferencePhase(enum.Enum):
    """``enum class InferencePhase`` (``phase_pipeline.h:24-28``)."""
    Prefill = 0
    Decode = 1
    Unknown = 2


@dataclass
class PhaseConfig:
    """Per-phase settings (``struct PhaseConfig``, ``phase_pipeline.h:31-53``), reduced to what
    concerns the quantised operator.

    ``matmul_strategy``  ``"gemv"`` (the reference's "vecmat"), ``"gemm"`` (its "tiled64") or
                         ``"auto"``: advisory, as in the reference;
    ``gemv_max_m``       largest M that takes the decode kernels while this phase is active
                         (1..32), or 0 to let the library choose per problem (16 or 32 by
                         weight format; up to 64 for bf16 activations with group-wise scales);
    ``capture_graph``    replay the step from a CUDA graph (the counterpart of the reference's
                         ``encoder_max_ops`` / ``auto_flush_threshold`` command batching)."""
    matmul_strategy: str = "auto"
    gemv_max_m: int = 0
    capture_graph: bool = False

    def validate(self) -> None:
        if self.matmul_strategy not in MATMUL_STRATEGIES:
            raise ValueError(f"matmul_strategy must be one of {MATMUL_STRATEGIES}")
        if not 0 <= int(self.gemv_max_m) <= 32:
            raise ValueError("gemv_max_m must be in 0..32")


def detect_phase(batch_size: int, seq_len: int) -> InferencePhase:
    """The reference's heuristic (``phase_pipeline.mm:42-51``): one token per sequence, or at
    most four tokens of a single sequence, is decode; everything else prefill."""
    if seq_len == 1 or (seq_len <= 4 and batch_size == 1):
        return InferencePhase.Decode
    return InferencePhase.Prefill


class PhasePipeline:
    """Keeps a prefill and a decode configuration and applies the active one.

    ``backend`` is the module that holds ``set_option`` / ``get_option`` (``metal_native._C``);
    it is imported on first use so that building a pipeline, detecting phases and editing
    configurations need no GPU and no library."""

    def __init__(self, backend=None):
        self._backend = backend
        self._lock = threading.Lock()
        self._phase = InferencePhase.Unknown
        # phase_pipeline.mm:27-40: tiled kernel for prefill, vecmat for decode
        self._prefill = PhaseConfig(matmul_strategy="gemm", gemv_max_m=0, capture_graph=False)
        self._decode = PhaseConfig(matmul_strategy="gemv", gemv_max_m=0, capture_graph=True)

    # -- phase management (phase_pipeline.mm:76-89)
    def set_phase(self, phase: InferencePhase) -> None:
        with self._lock:
            self._phase = InferencePhase(phase)

    def auto_detect_phase(self, batch_size: int, seq_len: int) -> InferencePhase:
        with self._lock:
            self._phase = detect_phase(batch_size, seq_len)
            return self._phase

    def current_phase(self) -> InferencePhase:
        with self._lock:
            return self._phase

    # -- configuration access and update (phase_pipeline.mm:91-114)
    def prefill_config(self) -> PhaseConfig:
        with self._lock:
            return replace(self._prefill)

    def decode_config(self) -> PhaseConfig:
        with self._lock:
            return replace(self._decode)

    def active_config(self) -> PhaseConfig:
        """Unknown falls back to the prefill configuration (``phase_pipeline.mm:53-63``)."""
        with self._lock:
            return replace(self._decode if self._phase is InferencePhase.Decode else self._prefill)

    def set_prefill_config(self, config: PhaseConfig) -> None:
        config.validate()
        with self._lock:
            self._prefill = replace(config)

    def set_decode_config(self, config: PhaseConfig) -> None:
        config.validate()
        with self._lock:
            self._decode = replace(config)

    # -- application (the reference's apply_to_pipeline, phase_pipeline.mm:167-)
    def _lib(self):
        if self._backend is None:
            from . import _C
            self._backend = _C
        return self._backend

    def apply(self) -> PhaseConfig:
        """Makes the active configuration the library's: sets the decode / tensor-core
        threshold.  Returns the configuration applied."""
        cfg = self.active_config()
        self._lib().set_option("gemv_max_m", cfg.gemv_max_m)
        return cfg

    def strategy_for(self, M: int) -> str:
        """Kernel family the applied threshold sends M tokens to: "gemv" or "gemm" (problems
        neither family takes fall to the any-shape kernel whatever the phase); "auto" where the
        threshold is left to the library and M lies between its smallest and largest choice
        (``select_path`` answers for a concrete problem)."""
        limit = self.active_config().gemv_max_m
        if limit == 0:
            return "gemv" if M <= 16 else "gemm" if M > 64 else "auto"
        return "gemv" if M <= limit else "gemm"

    def capture_step(self, step, warmup: int = 2):
        """Records ``step()`` (operator calls on the current device, with fixed tensors) into a
        CUDA graph and returns a function that replays it; when the active configuration does
        not ask for capture, returns ``step`` itself.  The first calls run eagerly: the allocation-
        free entry point and the kernels' one-time set-up must happen before capture."""
        cfg = self.apply()
        if not cfg.capture_graph:
            return step
        import torch
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(max(1, warmup)):
                step()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
        torch.cuda.current_stream().wait_stream(stream)
        return graph.replay
