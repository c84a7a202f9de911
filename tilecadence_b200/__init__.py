"""B200-native attention hot path with TileCadence's operator surface.

Modules mirror the reference package: ``placement`` (handoff planner), ``operator`` (schedule
emitter), ``model`` / ``exchange`` / ``emit_exchange`` (two-tile exchange planner and emitter),
``cuda_runtime`` (build + load), ``bench_operator`` / ``bench_exchange`` (verification and timing
harnesses), plus ``sharding`` for the single-node multi-GPU drivers.
"""
__version__ = "0.1.0"
