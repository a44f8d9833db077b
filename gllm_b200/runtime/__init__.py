"""Runtime heuristics: measured buckets, sub-batching, epilogue telemetry, variant registry, director, sensors."""
from .buckets import GoldenBuckets, LatencyProbe, LogHistogram  # noqa: F401
from .director import ConsensusDetector, ConsensusEvent, DecayingReservoir, Director, DirectorSharedState  # noqa: F401
from .epilogue import (Advice, EpilogueAggregator, EpilogueSignal, GateSkipMode, SinkTracker, gate_skip_decision,  # noqa: F401
                       signals_from_tensors)
from .sensors import SystemTopology, derive_constraints, host_memory_pressure, probe_system, read_meminfo  # noqa: F401
from .sub_batch import ShapeClass, classify, compact, run_ragged, scatter_back, sub_batches  # noqa: F401
from .variants import BudgetExceeded, CodeSection, CompiledVariant, MechanismId, VariantKey, VariantRegistry  # noqa: F401
