"""Build and load the sm_100a C-ABI library behind the reference's operator interface.

Mirrors ``tilecadence/cuda_runtime.py`` (``cuda_device`` :63-75, ``build_cuda`` :78-146): a
directory emitted by :mod:`tilecadence_b200.operator` is compiled for the GPU and returned as an
object with ``forward_out`` / ``workspace_spec`` / ``resources`` plus a build receipt. Differences
that follow from the B200-only design:

* the target is always ``compute_100a``/``sm_100a``; a device of any other generation is rejected;
* the library is a plain shared object with ``extern "C"`` entry points loaded through ``ctypes``
  (no torch C++ extension, no dispatcher namespace); tensors are validated here exactly as the
  reference's host code does (``cuda/prefill/common.cuh:36-60``, ``cuda/decode/decode.cu:38-60,
  158-179``) and passed down as raw pointers on torch's current stream;
* builds are cached inside the package tree under ``_build/`` keyed by the hash of every source
  file and flag, so a library compiled on a machine without a GPU is reused on the GPU box;
* no FlashAttention / CUTLASS checkout is needed; ``flash_attention_root`` is accepted and ignored.

There is no CPU path: if the library cannot be built or loaded the calls raise.
"""
from __future__ import annotations

import ctypes
from hashlib import sha256
import json
import os
from pathlib import Path
import shutil
import subprocess
import threading

PACKAGE_ROOT = Path(__file__).resolve().parent
CSRC = PACKAGE_ROOT / "csrc"
INCLUDE = PACKAGE_ROOT.parent / "include"
BUILD_DIR = PACKAGE_ROOT / "_build"
TARGET = "sm_100a"
CUDA_FLAGS = (
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-shared",
)
SOURCE_SUFFIXES = (".cu", ".cuh", ".h", ".hpp", ".cpp")
PHASES = ("prefill", "decode", "exchange")

_lock = threading.Lock()
_loaded: dict[str, "Library"] = {}


def file_sha256(path):
    """Hex SHA-256 of a file's bytes."""
    import hashlib

    with open(path, "rb") as stream:
        return hashlib.file_digest(stream, "sha256").hexdigest()


def find_nvcc():
    """Path of nvcc: ``$CUDA_HOME/bin`` (or ``$CUDA_PATH``, or /usr/local/cuda) first, then ``$PATH``."""
    roots = [os.environ.get(name) for name in ("CUDA_HOME", "CUDA_PATH")] + ["/usr/local/cuda"]
    for root in roots:
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return Path(root) / "bin" / "nvcc"
    on_path = shutil.which("nvcc")
    return Path(on_path) if on_path else None


def cuda_device(device="cuda:0"):
    """``(torch.device with an explicit index, compute capability)`` of a usable sm_100 device; anything
    else (no CUDA build of torch, no visible GPU, another architecture) is a ``RuntimeError``: there is
    no other code path to fall back to."""
    import torch

    wanted = torch.device(device)
    usable = wanted.type == "cuda" and bool(torch.version.cuda) and torch.cuda.is_available()
    if not usable:
        raise RuntimeError("An NVIDIA CUDA device and CUDA-enabled PyTorch are required")
    if wanted.index is None:
        wanted = torch.device("cuda", torch.cuda.current_device())
    major, minor = torch.cuda.get_device_capability(wanted)
    if major != 10:
        raise RuntimeError(f"The kernels are written for sm_100a only; device reports sm_{major}{minor}")
    return wanted, (major, minor)


def staged_sources(phase):
    """Flat {name: path} view of what an emitted directory for one phase contains."""
    files = {"tilecadence_b200.h": INCLUDE / "tilecadence_b200.h"}
    for directory in ("common", phase):
        for path in sorted((CSRC / directory).iterdir()):
            if path.is_file() and path.suffix in SOURCE_SUFFIXES:
                files[path.name] = path
    return files


def _compile(units, include_dirs, files, verbose=False, defines=()):
    """Compile ``units`` into one cached shared object; needs nvcc but no GPU.

    The cache key covers the named source files, the flags and the ``defines`` (preprocessor symbols for
    diagnostic builds) only, so a library built on a machine without a GPU is found again on the GPU
    machine from the same sources.
    """
    compiler = "unknown"
    nvcc = find_nvcc()
    if nvcc is not None:
        compiler = subprocess.check_output([str(nvcc), "--version"], text=True).strip().splitlines()[-1]
    identity = {
        "source_sha256": {name: file_sha256(path) for name, path in sorted(files.items())},
        "target": TARGET,
        "cuda_flags": list(CUDA_FLAGS) + [f"-D{symbol}" for symbol in defines],
    }
    key = sha256(json.dumps(identity, sort_keys=True).encode()).hexdigest()[:20]
    identity["cuda_compiler"] = compiler
    name = "tilecadence_" + key
    library = BUILD_DIR / f"lib{name}.so"
    with _lock:
        if not library.is_file():
            if nvcc is None:
                raise RuntimeError("Set CUDA_HOME to an installed CUDA Toolkit with nvcc: no prebuilt library "
                                   f"matches these sources ({library.name})")
            BUILD_DIR.mkdir(parents=True, exist_ok=True)
            temporary = library.with_name(f"{library.stem}.{os.getpid()}.tmp.so")
            command = [str(nvcc), *CUDA_FLAGS, *(f"-D{symbol}" for symbol in defines)]
            if verbose:
                command.append("-Xptxas=-v")
            for directory in include_dirs:
                command += ["-I", str(directory)]
            command += [*map(str, units), "-o", str(temporary)]
            result = subprocess.run(command, capture_output=True, text=True)
            if result.returncode != 0:
                raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
            if verbose:
                print(result.stderr)
            os.replace(temporary, library)
    identity.update(module=name, module_path=str(library), module_sha256=file_sha256(library))
    return library, identity


def compile_directory(source_dir, verbose=False, defines=()):
    """Compile every .cu of a flat emitted directory. Returns ``(library_path, identity)``."""
    source_dir = Path(source_dir).resolve()
    files = {path.name: path for path in sorted(source_dir.iterdir())
             if path.is_file() and path.suffix in SOURCE_SUFFIXES}
    units = [path for path in files.values() if path.suffix == ".cu"]
    if not units:
        raise ValueError(f"No generated CUDA translation unit in {source_dir}")
    return _compile(units, [source_dir], files, verbose, defines)


def compile_tree(verbose=False):
    """Compile every phase from the in-tree sources (default offsets) into one library."""
    files = {"tilecadence_b200.h": INCLUDE / "tilecadence_b200.h"}
    units = []
    for folder in sorted(path for path in CSRC.iterdir() if path.is_dir()):
        for path in sorted(folder.iterdir()):
            if path.is_file() and path.suffix in SOURCE_SUFFIXES:
                files[f"{folder.name}/{path.name}"] = path
                if path.suffix == ".cu":
                    units.append(path)
    return _compile(units, [CSRC / "common", INCLUDE], files, verbose)


class Library:
    """ctypes view of one compiled C-ABI library."""

    SIGNATURES = {
        "tc_last_error": (ctypes.c_char_p, ()),
        "tc_abi_version": (ctypes.c_int, ()),
        "tc_device_status": (ctypes.c_int, (ctypes.c_int, ctypes.POINTER(ctypes.c_int32))),
        "tc_prefill_workspace_spec": (ctypes.c_int, (ctypes.c_int, *[ctypes.c_int64] * 5, ctypes.c_int,
                                                     ctypes.POINTER(ctypes.c_int64))),
        "tc_prefill_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p,
            ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64),
            ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_void_p,
            *[ctypes.c_int64] * 7, ctypes.c_double, ctypes.c_int)),
        "tc_prefill_key_split_workspace_bytes": (ctypes.c_int, (*[ctypes.c_int64] * 3, ctypes.POINTER(ctypes.c_int64))),
        "tc_prefill_key_split_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p,
            ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64),
            ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 4, ctypes.c_double, ctypes.c_int64,
            ctypes.POINTER(ctypes.c_int64))),
        "tc_prefill_resources": (ctypes.c_int, (
            ctypes.c_int, *[ctypes.POINTER(ctypes.c_int64)] * 3, *[ctypes.c_int64] * 5, ctypes.c_int,
            ctypes.POINTER(ctypes.c_int64), ctypes.c_int64, ctypes.POINTER(ctypes.c_int64))),
        "tc_decode_workspace_spec": (ctypes.c_int, (ctypes.c_int, *[ctypes.c_int64] * 5, ctypes.c_int,
                                                    ctypes.POINTER(ctypes.c_int64))),
        "tc_decode_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 5, ctypes.c_int)),
        "tc_decode_forward_out_flags": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 5, ctypes.c_int, ctypes.c_int64)),
        "tc_decode_forward_out_static": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, *[ctypes.c_int64] * 5, ctypes.c_int)),
        "tc_decode_partial_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 5, ctypes.c_int, ctypes.c_int64)),
        "tc_qkv_rope_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 6, ctypes.c_int64, *[ctypes.c_void_p] * 4,
            *[ctypes.c_int64] * 4, ctypes.c_double)),
        "tc_qkv_rope_forward_out_flags": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 6, ctypes.c_int64, *[ctypes.c_void_p] * 4,
            *[ctypes.c_int64] * 4, ctypes.c_double, ctypes.c_int)),
        "tc_decode_rope_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 5, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int64)),
        "tc_decode_indexed_forward_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 6, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_int64, ctypes.c_void_p)),
        "tc_decode_exchange_out": (ctypes.c_int, (
            ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 8, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, *[ctypes.c_int64] * 5, ctypes.c_int, *[ctypes.c_int64] * 3,
            ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64)),
        "tc_decode_static_status_word": (ctypes.c_int, (ctypes.c_int, ctypes.POINTER(ctypes.c_void_p))),
        "tc_peer_block_bytes": (ctypes.c_int, (*[ctypes.c_int64] * 3, ctypes.POINTER(ctypes.c_int64))),
        "tc_peer_block_create": (ctypes.c_int, (ctypes.c_int, ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p),
                                                ctypes.c_char_p)),
        "tc_peer_block_open": (ctypes.c_int, (ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p))),
        "tc_peer_block_close": (ctypes.c_int, (ctypes.c_int, ctypes.c_void_p)),
        "tc_peer_block_destroy": (ctypes.c_int, (ctypes.c_int, ctypes.c_void_p)),
        "tc_combine_partials": (ctypes.c_int, (ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               *[ctypes.c_int64] * 4, ctypes.c_void_p, ctypes.c_void_p)),
        "tc_exchange_forward_out": (ctypes.c_int, (ctypes.c_int, ctypes.c_void_p, *[ctypes.c_void_p] * 5,
                                                   ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int)),
        "tc_exchange_resources": (ctypes.c_int, (ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                 ctypes.POINTER(ctypes.c_int64))),
        "tc_decode_resources": (ctypes.c_int, (ctypes.c_int, *[ctypes.c_int64] * 5, ctypes.c_int,
                                               ctypes.POINTER(ctypes.c_int64), ctypes.c_int64,
                                               ctypes.POINTER(ctypes.c_int64))),
    }

    def __init__(self, path):
        self.path = Path(path)
        self.handle = ctypes.CDLL(str(self.path))
        self.symbols = set()
        self.functions = {}
        for name, (restype, argtypes) in self.SIGNATURES.items():
            try:
                function = getattr(self.handle, name)
            except AttributeError:
                continue
            function.restype = restype
            function.argtypes = list(argtypes)
            self.symbols.add(name)
            self.functions[name] = function
        if "tc_last_error" not in self.symbols:
            raise RuntimeError(f"{self.path} does not export the tilecadence_b200 C ABI")

    def has(self, prefix):
        return any(name.startswith(prefix) for name in self.symbols)

    def call(self, name, *arguments):
        function = self.functions.get(name)
        if function is None:
            raise RuntimeError(f"{self.path.name} does not export {name}; this library was built for another phase")
        status = function(*arguments)
        if status != 0:
            message = self.handle.tc_last_error().decode("utf-8", "replace")
            raise RuntimeError(f"{name}: {message} (status {status})")

    def device_status(self, device_index):
        value = ctypes.c_int32(0)
        self.call("tc_device_status", int(device_index), ctypes.byref(value))
        return value.value


def load_library(path):
    path = str(Path(path).resolve())
    with _lock:
        if path not in _loaded:
            _loaded[path] = Library(path)
        return _loaded[path]


def _strides(tensor):
    return (ctypes.c_int64 * 3)(tensor.stride(0), tensor.stride(1), tensor.stride(2))


def _stream(tensor):
    """torch's current stream on the tensor's device as a raw ``cudaStream_t`` value (0 = the default stream)."""
    import torch

    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:  # one C call instead of building a Stream object on every operator call
        return raw(tensor.device.index)
    return torch.cuda.current_stream(tensor.device).cuda_stream


def _require(condition, message):
    if not condition:
        raise RuntimeError(message)


def _pointer(tensor):
    """Device address as an integer; every entry point's argtypes declare the slot as a pointer."""
    return tensor.data_ptr()


class PrefillOps:
    """``forward_out`` / ``workspace_spec`` / ``resources`` with the reference's prefill schemas
    (``tilecadence/cuda/prefill/binding.cpp:11-13``). ``q_heads`` defaults to the reference's 32;
    a KV-head-group shard may pass its own count."""

    phase = "prefill"

    def __init__(self, library, q_heads=32):
        self.library = library
        self.q_heads = q_heads

    def _check_inputs(self, q, k, v, causal):
        import torch

        heads = self.q_heads
        _require(q.is_cuda and q.dim() == 4 and q.size(0) > 0 and q.size(1) > 0 and q.size(2) == heads
                 and q.size(3) == 128, f"Q must be actual CUDA BNHD[B,T,{heads},128]")
        for tensor in (q, k, v):
            _require(tensor.device == q.device and tensor.dtype == torch.bfloat16 and not tensor.requires_grad,
                     "Same-device inference BF16 Q/K/V required")
            _require(tensor.dim() == 4 and tensor.stride(3) == 1, "BNHD inputs must have contiguous last dimension only")
            _require(tensor.data_ptr() % 16 == 0, "Aligned native Q/K/V base required")
            for axis in range(3):
                _require(tensor.size(axis) == 1 or (tensor.stride(axis) >= 0 and tensor.stride(axis) % 8 == 0),
                         "Native vector row/head alignment requires strides divisible by8 elements")
        _require(k.size(0) == q.size(0) and k.size(1) > 0 and k.size(2) == heads // 4 and k.size(3) == 128
                 and v.shape == k.shape, f"Actual visible K/V must be BNHD[B,Tk,{heads // 4},128]")
        _require(bool(causal) and q.size(1) > 1 and q.size(1) == k.size(1), "Full causal no-past prefill requires Tq=Tk>1")

    def workspace_spec(self, q, k, v, num_splits, mapping, causal):
        self._check_inputs(q, k, v, causal)
        spec = (ctypes.c_int64 * 3)()
        self.library.call("tc_prefill_workspace_spec", q.device.index, q.size(0), q.size(1), q.size(2),
                          int(num_splits), int(mapping), int(bool(causal)), spec)
        return list(spec)

    def forward_out(self, q, k, v, out, lse, workspace_o, workspace_lse, num_splits, mapping, scale, causal):
        import torch

        self._check_inputs(q, k, v, causal)
        _require(out.device == q.device and out.dtype == q.dtype and out.shape == q.shape and out.is_contiguous()
                 and not out.requires_grad, "Common complete output must be contiguous BNHD with Q shape")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous() and not lse.requires_grad
                 and tuple(lse.shape) == (q.size(0), q.size(2), q.size(1)),
                 f"Complete natural-log LSE must be FP32[B,{q.size(2)},Tq]")
        _require(workspace_o.numel() == 0 and workspace_lse.numel() == 0, "Generated long prefill uses no split workspace")
        self.library.call(
            "tc_prefill_forward_out", q.device.index, _stream(q), _pointer(q), _strides(q), _pointer(k), _strides(k),
            _pointer(v), _strides(v), _pointer(out), _pointer(lse), 0, 0, q.size(0), q.size(1), q.size(2),
            int(num_splits), int(mapping), float(scale), int(bool(causal)))

    def bind_forward_out(self, q, k, v, out, lse, workspace_o, workspace_lse, num_splits, mapping, scale, causal):
        """Validate once and return a zero-argument callable that repeats this exact call (see
        :meth:`DecodeOps.bind_forward_out`)."""
        import torch

        self._check_inputs(q, k, v, causal)
        _require(out.device == q.device and out.dtype == q.dtype and out.shape == q.shape and out.is_contiguous()
                 and not out.requires_grad, "Common complete output must be contiguous BNHD with Q shape")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous() and not lse.requires_grad
                 and tuple(lse.shape) == (q.size(0), q.size(2), q.size(1)),
                 f"Complete natural-log LSE must be FP32[B,{q.size(2)},Tq]")
        _require(workspace_o.numel() == 0 and workspace_lse.numel() == 0, "Generated long prefill uses no split workspace")
        keep = (q, k, v, out, lse)
        tail = (_pointer(q), _strides(q), _pointer(k), _strides(k), _pointer(v), _strides(v), _pointer(out), _pointer(lse),
                0, 0, q.size(0), q.size(1), q.size(2), int(num_splits), int(mapping), float(scale), int(bool(causal)))
        function = self.library.handle.tc_prefill_forward_out
        library, probe = self.library, q

        def invoke(_keep=keep):
            status = function(probe.device.index, _stream(probe), *tail)
            if status != 0:
                raise RuntimeError("tc_prefill_forward_out: " + library.handle.tc_last_error().decode("utf-8", "replace"))

        return invoke

    def key_split_workspace_bytes(self, q):
        """Bytes of the uint8 workspace :meth:`key_split_forward_out` needs for ``q``'s geometry."""
        size = ctypes.c_int64(0)
        self.library.call("tc_prefill_key_split_workspace_bytes", q.size(0), q.size(1), q.size(2), ctypes.byref(size))
        return size.value

    def key_split_forward_out(self, q, k, v, out, lse, workspace, mapping, scale, key_splits=0):
        """Prefill with up to two CTAs per query tile (``tc_prefill_key_split_forward_out``): for launches that
        cannot fill the GPU otherwise, such as a KV-head-group shard. ``workspace`` is a uint8 CUDA tensor of
        :meth:`key_split_workspace_bytes` bytes. Returns the number of key splits used (1 or 2)."""
        import torch

        self._check_inputs(q, k, v, True)
        _require(out.device == q.device and out.dtype == q.dtype and out.shape == q.shape and out.is_contiguous()
                 and not out.requires_grad, "Common complete output must be contiguous BNHD with Q shape")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous() and not lse.requires_grad
                 and tuple(lse.shape) == (q.size(0), q.size(2), q.size(1)),
                 f"Complete natural-log LSE must be FP32[B,{q.size(2)},Tq]")
        _require(workspace.device == q.device and workspace.dtype == torch.uint8 and workspace.is_contiguous(),
                 "Contiguous CUDA uint8 workspace required")
        used = ctypes.c_int64(0)
        self.library.call(
            "tc_prefill_key_split_forward_out", q.device.index, _stream(q), _pointer(q), _strides(q), _pointer(k),
            _strides(k), _pointer(v), _strides(v), _pointer(out), _pointer(lse), _pointer(workspace), workspace.numel(),
            q.size(0), q.size(1), q.size(2), int(mapping), float(scale), int(key_splits), ctypes.byref(used))
        return used.value

    def resources(self, q, k, v, num_splits, mapping, causal):
        self._check_inputs(q, k, v, causal)
        values = (ctypes.c_int64 * 64)()
        count = ctypes.c_int64(0)
        self.library.call("tc_prefill_resources", q.device.index, _strides(q), _strides(k), _strides(v), q.size(0),
                          q.size(1), q.size(2), int(num_splits), int(mapping), int(bool(causal)), values, 64,
                          ctypes.byref(count))
        return list(values[:count.value])


#: ``flags`` bits of ``tc_decode_forward_out_flags``; same values as TC_DECODE_CACHE_STABLE and
#: TC_DECODE_PREFIX_STABLE in the header.
DECODE_CACHE_STABLE = 1
DECODE_PREFIX_STABLE = 2
#: ``flags`` bit of ``tc_qkv_rope_forward_out_flags`` (TC_PROJECT_RELEASE_EARLY in the header).
PROJECT_RELEASE_EARLY = 1


def _decode_flags(cache_stable):
    if cache_stable == "prefix":
        return DECODE_PREFIX_STABLE
    _require(cache_stable is True, 'cache_stable must be False, True or "prefix"')
    return DECODE_CACHE_STABLE


class DecodeOps:
    """``forward_out`` / ``workspace_spec`` / ``resources`` with the reference's decode schemas
    (``tilecadence/cuda/decode/binding.cpp:17-24``), plus the sharded ``partial_out`` and
    ``combine_partials`` used by the multi-GPU driver."""

    phase = "decode"

    def __init__(self, library, q_heads=32):
        self.library = library
        self.q_heads = q_heads

    def _check_q_cache_lengths(self, q, cache, lengths):
        import torch

        heads = self.q_heads
        device = q.device
        _require(q.is_cuda and cache.device == device and lengths.device == device,
                 "Q/cache/old_lengths must be CUDA on the same device")
        q_shape, cache_shape = q.shape, cache.shape  # one call each: these checks run on every decode step
        _require(len(q_shape) == 4 and q_shape[0] > 0 and q_shape[1] == 1 and q_shape[2] == heads and q_shape[3] == 128,
                 f"Q must be [B,1,{heads},128]")
        _require(len(cache_shape) == 4 and cache_shape[0] == q_shape[0] and cache_shape[1] >= 4
                 and cache_shape[2] == heads // 4 and cache_shape[3] == 128,
                 f"Full capacity cache must be [B,C>=4,{heads // 4},128]")
        _require(q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and q.is_contiguous()
                 and cache.is_contiguous() and not q.requires_grad and not cache.requires_grad,
                 "Contiguous BF16 inference Q and FULL capacity cache required")
        _require(lengths.dtype == torch.int32 and lengths.is_contiguous() and lengths.shape == (q_shape[0],)
                 and not lengths.requires_grad, "old_lengths must be contiguous CUDA int32[B]")
        _require(q.data_ptr() % 16 == 0 and cache.data_ptr() % 16 == 0, "16-byte aligned Q/cache required")

    def workspace_spec(self, q, kcache, old_lengths, num_splits, mapping, append):
        self._check_q_cache_lengths(q, kcache, old_lengths)
        spec = (ctypes.c_int64 * 3)()
        self.library.call("tc_decode_workspace_spec", q.device.index, q.size(0), kcache.size(1), kcache.size(2),
                          int(num_splits), int(mapping), int(bool(append)), spec)
        return list(spec)

    def _check_call(self, q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse):
        import torch

        self._check_q_cache_lengths(q, kcache, old_lengths)
        device, dtype = q.device, q.dtype
        _require(vcache.device == device and vcache.shape == kcache.shape and vcache.dtype == dtype
                 and vcache.is_contiguous() and not vcache.requires_grad, "Vcache must match FULL contiguous BF16 Kcache")
        new_shape = (q.shape[0], 1, kcache.shape[2], 128)
        for tensor in (knew, vnew):
            _require(tensor.device == device and tensor.dtype == dtype and tensor.shape == new_shape
                     and tensor.is_contiguous() and not tensor.requires_grad,
                     "knew/vnew must be contiguous BF16[B,1,Hkv,128]")
        for workspace in (workspace_o, workspace_lse):
            _require(workspace.device == device and workspace.dtype == torch.float32
                     and workspace.is_contiguous() and not workspace.requires_grad,
                     "Contiguous CUDA FP32 workspace required")

    @staticmethod
    def _check_out(q, out, lse):
        import torch

        _require(out.device == q.device and out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous()
                 and not out.requires_grad, "Invalid complete output")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous()
                 and tuple(lse.shape) == (q.size(0), q.size(2), 1) and not lse.requires_grad, "Invalid full float32 LSE")

    def forward_out(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse,
                    num_splits, mapping, append, *, cache_stable=False):
        """One decode step. ``cache_stable=True`` is the caller's promise that the kernel enqueued just
        before this call writes neither the caches' visible rows nor ``old_lengths``; the K/V stream then
        starts while that kernel is still finishing (``TC_DECODE_CACHE_STABLE``). ``cache_stable="prefix"``
        is the narrower promise for a preceding kernel that was the previous decode step of the same caches
        and appended row ``old_lengths - 1`` (``TC_DECODE_PREFIX_STABLE``)."""
        self._check_call(q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse)
        self._check_out(q, out, lse)
        arguments = (
            q.device.index, _stream(q), _pointer(q), _pointer(kcache), _pointer(vcache),
            _pointer(knew), _pointer(vnew), _pointer(old_lengths), _pointer(out), _pointer(lse),
            _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse), workspace_lse.numel(),
            q.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping), int(bool(append)))
        if cache_stable:
            self.library.call("tc_decode_forward_out_flags", *arguments, _decode_flags(cache_stable))
        else:
            self.library.call("tc_decode_forward_out", *arguments)

    def bind_forward_out(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse,
                         num_splits, mapping, append, *, cache_stable=False):
        """Validate once and return a zero-argument callable that repeats this exact call.

        A decode step on a short cache takes a few microseconds on the GPU, less than the tensor
        checks cost in Python; a serving loop that reuses its buffers binds the call once. The
        callable launches on torch's current stream at the time it is invoked.
        """
        import torch

        self._check_call(q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse)
        _require(out.device == q.device and out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous()
                 and not out.requires_grad, "Invalid complete output")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous()
                 and tuple(lse.shape) == (q.size(0), q.size(2), 1) and not lse.requires_grad, "Invalid full float32 LSE")
        keep = (q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse)
        head = (q.device.index,)
        tail = (_pointer(q), _pointer(kcache), _pointer(vcache), _pointer(knew), _pointer(vnew), _pointer(old_lengths),
                _pointer(out), _pointer(lse), _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse),
                workspace_lse.numel(), q.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping),
                int(bool(append)))
        if cache_stable:
            function, tail = self.library.handle.tc_decode_forward_out_flags, tail + (_decode_flags(cache_stable),)
        else:
            function = self.library.handle.tc_decode_forward_out
        library, probe = self.library, q

        def invoke(_keep=keep):
            status = function(*head, _stream(probe), *tail)
            if status != 0:
                raise RuntimeError("tc_decode_forward_out: " + library.handle.tc_last_error().decode("utf-8", "replace"))

        return invoke

    def partial_out(self, q, kcache, vcache, knew, vnew, old_lengths, partial_o, partial_lse, workspace_o,
                    workspace_lse, num_splits, mapping, append, kv_shard_start):
        import torch

        self._check_call(q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse)
        rows = q.size(0) * q.size(2)
        _require(partial_o.device == q.device and partial_o.dtype == torch.float32 and partial_o.is_contiguous()
                 and partial_o.numel() == rows * 128, "partial O must be contiguous FP32[B,Hq,128]")
        _require(partial_lse.device == q.device and partial_lse.dtype == torch.float32 and partial_lse.is_contiguous()
                 and partial_lse.numel() == rows, "partial LSE must be contiguous FP32[B,Hq]")
        self.library.call(
            "tc_decode_partial_out", q.device.index, _stream(q), _pointer(q), _pointer(kcache), _pointer(vcache),
            _pointer(knew), _pointer(vnew), _pointer(old_lengths), _pointer(partial_o), _pointer(partial_lse),
            _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse), workspace_lse.numel(),
            q.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping), int(bool(append)),
            int(kv_shard_start))

    def rope_forward_out(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse,
                         num_splits, mapping, append, rope_cos, rope_sin):
        """``forward_out`` for un-rotated ``q`` / ``knew``: rotary position embedding (rotate-half, tables
        FP32 [positions, 64], row = ``old_lengths[b]``) is applied inside the decode launch and the rotated K
        row is what gets appended."""
        import torch

        self._check_call(q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse)
        self._check_out(q, out, lse)
        for table in (rope_cos, rope_sin):
            _require(table.device == q.device and table.dtype == torch.float32 and table.dim() == 2
                     and table.size(1) == 64 and table.is_contiguous() and table.shape == rope_cos.shape,
                     "RoPE tables must be contiguous FP32[positions,64]")
        self.library.call(
            "tc_decode_rope_forward_out", q.device.index, _stream(q), _pointer(q), _pointer(kcache), _pointer(vcache),
            _pointer(knew), _pointer(vnew), _pointer(old_lengths), _pointer(out), _pointer(lse),
            _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse), workspace_lse.numel(),
            q.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping), int(bool(append)),
            _pointer(rope_cos), _pointer(rope_sin), rope_cos.size(0))

    def indexed_forward_out(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse,
                            num_splits, mapping, append, block_table=None, cache_batch_idx=None):
        """Decode step over paged caches (``block_table`` int32 [B, pages_per_seq]; caches
        [pages, page_size, Hkv, 128]) or over caches whose batch entry is picked per sequence
        (``cache_batch_idx`` int32 [B]). The workspace is sized as for a contiguous cache of the
        sequence capacity: ``workspace_spec`` takes any tensor of shape [B, capacity, Hkv, 128]-like
        geometry, see :meth:`indexed_workspace_spec`."""
        import torch

        _require((block_table is None) != (cache_batch_idx is None), "pass exactly one of block_table / cache_batch_idx")
        _require(q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4 and q.size(1) == 1 and q.size(3) == 128
                 and q.size(2) == self.q_heads and q.is_contiguous(), "Q must be contiguous BF16[B,1,Hq,128]")
        _require(kcache.device == q.device and kcache.dtype == q.dtype and kcache.dim() == 4 and kcache.size(3) == 128
                 and kcache.size(2) * 4 == q.size(2) and kcache.is_contiguous() and vcache.shape == kcache.shape
                 and vcache.device == q.device and vcache.dtype == q.dtype and vcache.is_contiguous(),
                 "caches must be contiguous BF16[slots,rows,Hkv,128]")
        for tensor in (knew, vnew):
            _require(tensor.device == q.device and tensor.dtype == q.dtype and tensor.is_contiguous()
                     and tuple(tensor.shape) == (q.size(0), 1, kcache.size(2), 128), "knew/vnew must be BF16[B,1,Hkv,128]")
        _require(old_lengths.device == q.device and old_lengths.dtype == torch.int32 and old_lengths.is_contiguous()
                 and tuple(old_lengths.shape) == (q.size(0),), "old_lengths must be contiguous int32[B]")
        for workspace in (workspace_o, workspace_lse):
            _require(workspace.is_cuda and workspace.device == q.device and workspace.dtype == torch.float32
                     and workspace.is_contiguous(), "Contiguous CUDA FP32 workspace required")
        self._check_out(q, out, lse)
        index = block_table if block_table is not None else cache_batch_idx
        _require(index.device == q.device and index.dtype == torch.int32 and index.size(0) == q.size(0)
                 and index.dim() == (2 if block_table is not None else 1) and index.stride(-1) == 1,
                 "block_table must be int32[B,pages] / cache_batch_idx int32[B] with a contiguous last dimension")
        pages = block_table.size(1) if block_table is not None else 0
        self.library.call(
            "tc_decode_indexed_forward_out", q.device.index, _stream(q), _pointer(q), _pointer(kcache), _pointer(vcache),
            _pointer(knew), _pointer(vnew), _pointer(old_lengths), _pointer(out), _pointer(lse),
            _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse), workspace_lse.numel(),
            q.size(0), kcache.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping), int(bool(append)),
            _pointer(block_table) if block_table is not None else None,
            block_table.stride(0) if block_table is not None else 0, pages,
            _pointer(cache_batch_idx) if cache_batch_idx is not None else None)

    def indexed_workspace_spec(self, batch, capacity, kv_heads, device_index, num_splits=0, mapping=1, append=True):
        """``[splits, workspace_o elements, workspace_lse elements]`` for a sequence capacity."""
        spec = (ctypes.c_int64 * 3)()
        self.library.call("tc_decode_workspace_spec", int(device_index), int(batch), int(capacity), int(kv_heads),
                          int(num_splits), int(mapping), int(bool(append)), spec)
        return list(spec)

    def exchange_out(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, workspace_o, workspace_lse,
                     num_splits, mapping, append, kv_shard_start, rank, peer_blocks, peer_block_bytes):
        """Sharded decode step with the cross-GPU merge inside the launch; ``peer_blocks`` is the
        ctypes array of every rank's exchange block (see :class:`tilecadence_b200.sharding.PeerBlocks`)
        and ``peer_block_bytes`` the size each of them was created with."""
        self._check_call(q, kcache, vcache, knew, vnew, old_lengths, workspace_o, workspace_lse)
        self._check_out(q, out, lse)
        self.library.call(
            "tc_decode_exchange_out", q.device.index, _stream(q), _pointer(q), _pointer(kcache), _pointer(vcache),
            _pointer(knew), _pointer(vnew), _pointer(old_lengths), _pointer(out), _pointer(lse),
            _pointer(workspace_o), workspace_o.numel(), _pointer(workspace_lse), workspace_lse.numel(),
            q.size(0), kcache.size(1), kcache.size(2), int(num_splits), int(mapping), int(bool(append)),
            int(kv_shard_start), len(peer_blocks), int(rank), peer_blocks, int(peer_block_bytes))

    def combine_partials(self, partial_o, partial_lse, out, lse):
        """Merge partial_o [parts, rows, 128] / partial_lse [parts, rows] (fp32; the part dimension may be
        strided, e.g. views into one gathered buffer) into out BF16 [rows*128] and lse FP32 [rows]."""
        import torch

        parts, rows = partial_lse.size(0), partial_lse[0].numel()
        _require(partial_o.is_cuda and partial_o.dtype == torch.float32 and partial_lse.dtype == torch.float32
                 and partial_o.size(0) == parts and partial_o[0].numel() == rows * 128
                 and partial_o[0].is_contiguous() and partial_lse[0].is_contiguous(),
                 "partials must be FP32 [parts,rows,128] / [parts,rows] with contiguous parts")
        _require(out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == rows * 128
                 and lse.dtype == torch.float32 and lse.is_contiguous() and lse.numel() == rows,
                 "combined O must be BF16[rows,128] and LSE FP32[rows]")
        stride_o = partial_o.stride(0) if parts > 1 else rows * 128
        stride_lse = partial_lse.stride(0) if parts > 1 else rows
        self.library.call("tc_combine_partials", partial_o.device.index, _stream(partial_o), _pointer(partial_o),
                          _pointer(partial_lse), parts, rows, stride_o, stride_lse, _pointer(out), _pointer(lse))

    def resources(self, q, kcache, old_lengths, num_splits, mapping, append):
        self._check_q_cache_lengths(q, kcache, old_lengths)
        values = (ctypes.c_int64 * 64)()
        count = ctypes.c_int64(0)
        self.library.call("tc_decode_resources", q.device.index, q.size(0), kcache.size(1), kcache.size(2),
                          int(num_splits), int(mapping), int(bool(append)), values, 64, ctypes.byref(count))
        return list(values[:count.value])


class ExchangeOps:
    """``forward_out`` / ``forward`` / ``resources`` with the reference's two-tile schemas
    (``tilecadence/cuda/exchange/binding.cpp:32-72,79-81``). q/k/v/out are contiguous [B,64,H,128] FP16 or
    BF16, lse FP32 [B,H,64]. ``nonce`` is accepted for signature compatibility; these plans need none."""

    phase = "exchange"

    def __init__(self, library):
        self.library = library

    def _check(self, q, k, v):
        import torch

        _require(q.is_cuda and q.dim() == 4 and q.size(0) > 0 and q.size(1) == 64 and q.size(2) > 0 and q.size(3) == 128,
                 "Q must be CUDA [B,64,H,128]")
        _require(q.dtype in (torch.float16, torch.bfloat16), "FP16 or BF16 inputs required")
        for tensor in (q, k, v):
            _require(tensor.device == q.device and tensor.dtype == q.dtype and tensor.shape == q.shape
                     and tensor.is_contiguous() and not tensor.requires_grad,
                     "Q, K and V must be contiguous same-shape inference tensors on one device")

    def forward_out(self, q, k, v, out, lse, nonce, causal, nonce_is_zero=True, diagnostic_non_nan_asserted=False):
        import torch

        self._check(q, k, v)
        _require(bool(nonce_is_zero) and not diagnostic_non_nan_asserted, "These plans take a zero nonce and no diagnostic guard")
        _require(out.device == q.device and out.dtype == q.dtype and out.shape == q.shape and out.is_contiguous()
                 and not out.requires_grad, "Output must be contiguous with Q's shape and dtype")
        _require(lse.device == q.device and lse.dtype == torch.float32 and lse.is_contiguous()
                 and tuple(lse.shape) == (q.size(0), q.size(2), 64), "LSE must be FP32 [B,H,64]")
        self.library.call("tc_exchange_forward_out", q.device.index, _stream(q), _pointer(q), _pointer(k), _pointer(v),
                          _pointer(out), _pointer(lse), q.size(0), q.size(2), int(q.dtype == torch.float16),
                          int(bool(causal)))

    def forward(self, q, k, v, nonce, causal, nonce_is_zero=True, diagnostic_non_nan_asserted=False):
        import torch

        out = torch.empty_like(q)
        lse = torch.empty((q.size(0), q.size(2), 64), device=q.device, dtype=torch.float32)
        self.forward_out(q, k, v, out, lse, nonce, causal, nonce_is_zero, diagnostic_non_nan_asserted)
        return [out, lse]

    def resources(self, q, causal):
        import torch

        values = (ctypes.c_int64 * 14)()
        self.library.call("tc_exchange_resources", q.device.index, int(q.dtype == torch.float16), int(bool(causal)), values)
        return list(values)


class ProjectOps:
    """The step before decode attention: fused QKV projection, per-head RMS norm and RoPE for one new
    token per sequence (``tc_qkv_rope_forward_out``). The reference has no such operator; its decode op
    takes the results as inputs."""

    phase = "project"

    def __init__(self, library, q_heads=32, kv_heads=8):
        self.library, self.q_heads, self.kv_heads = library, q_heads, kv_heads

    def forward_out(self, x, w_qkv, positions, q_out, knew_out, vnew_out, q_norm_weight=None, k_norm_weight=None,
                    rope_cos=None, rope_sin=None, rms_eps=1e-6, *, release_early=False):
        """``release_early=True`` (``TC_PROJECT_RELEASE_EARLY``) lets the kernel launched after this one start its
        independent part while the kernel launched before this one is still running; the caller promises that this
        is safe (it always is when the follower is another projection)."""
        import torch

        tokens, hidden = x.shape
        rows = (self.q_heads + 2 * self.kv_heads) * 128
        _require(x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and 1 <= tokens <= 8,
                 "x must be contiguous CUDA BF16[tokens<=8,hidden]")
        _require(w_qkv.device == x.device and w_qkv.dtype == x.dtype and w_qkv.is_contiguous()
                 and tuple(w_qkv.shape) == (rows, hidden), "w_qkv must be contiguous BF16[(Hq+2Hkv)*128,hidden]")
        for tensor, heads in ((q_out, self.q_heads), (knew_out, self.kv_heads), (vnew_out, self.kv_heads)):
            _require(tensor.device == x.device and tensor.dtype == x.dtype and tensor.is_contiguous()
                     and tuple(tensor.shape) == (tokens, 1, heads, 128), "outputs must be BF16[tokens,1,heads,128]")
        for weight in (q_norm_weight, k_norm_weight):
            _require(weight is None or (weight.device == x.device and weight.dtype == x.dtype
                                        and tuple(weight.shape) == (128,) and weight.is_contiguous()),
                     "norm weights must be BF16[128]")
        _require((rope_cos is None) == (rope_sin is None), "pass both RoPE tables or neither")
        if rope_cos is not None:
            for table in (rope_cos, rope_sin):
                _require(table.device == x.device and table.dtype == torch.float32 and table.dim() == 2
                         and table.size(1) == 64 and table.is_contiguous() and table.shape == rope_cos.shape,
                         "RoPE tables must be contiguous FP32[positions,64]")
            _require(positions is not None and positions.device == x.device and positions.dtype == torch.int32
                     and tuple(positions.shape) == (tokens,) and positions.is_contiguous(),
                     "positions must be contiguous int32[tokens]")
        optional = lambda tensor: _pointer(tensor) if tensor is not None else None
        arguments = (
            x.device.index, _stream(x), _pointer(x), _pointer(w_qkv),
            optional(q_norm_weight), optional(k_norm_weight), optional(rope_cos), optional(rope_sin),
            rope_cos.size(0) if rope_cos is not None else 0, optional(positions), _pointer(q_out), _pointer(knew_out),
            _pointer(vnew_out), tokens, hidden, self.q_heads, self.kv_heads, float(rms_eps))
        if release_early:
            self.library.call("tc_qkv_rope_forward_out_flags", *arguments, PROJECT_RELEASE_EARLY)
        else:
            self.library.call("tc_qkv_rope_forward_out", *arguments)


def ops_for(library, phase=None, q_heads=32):
    if phase is None:
        phase = ("prefill" if library.has("tc_prefill_") else "decode" if library.has("tc_decode_")
                 else "exchange" if library.has("tc_exchange_") else None)
    if phase == "exchange":
        return ExchangeOps(library)
    if phase == "prefill":
        return PrefillOps(library, q_heads)
    if phase == "decode":
        return DecodeOps(library, q_heads)
    if phase == "project":
        return ProjectOps(library, q_heads, q_heads // 4)
    raise RuntimeError(f"{library.path} exports neither the prefill nor the decode operator")


def build_cuda(source_dir, flash_attention_root=None, device="cuda:0"):
    """Return the operator object for an emitted directory and its reproducible build metadata."""
    import torch

    device, _ = cuda_device(device)
    library_path, identity = compile_directory(source_dir)
    library = load_library(library_path)
    receipt = {
        **identity,
        "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "device_name": torch.cuda.get_device_name(device),
        "device_index": device.index,
    }
    return ops_for(library), receipt


def default_library():
    """The combined library (every phase) built from the in-tree sources with default offsets."""
    library_path, _ = compile_tree()
    return load_library(library_path)


def default_ops(phase, q_heads=32):
    return ops_for(default_library(), phase, q_heads)
