"""B200-native attention hot path with TileCadence's operator surface.

Modules mirror the reference package: ``placement`` (handoff planner), ``operator`` (schedule
emitter), ``cuda_runtime`` (build + load), ``bench_operator`` (verification and timing harness),
plus ``sharding`` for the single-node multi-GPU drivers.
"""
__version__ = "0.1.0"
