"""ctypes binding of libtriturus_b200.so and its registration as torch custom ops.

The shared library is the product: there is no Python, Triton or CPU fallback behind these functions.  If
the library cannot be loaded the import fails loudly, and calling an op with tensors that are not on a
CUDA device raises.
"""

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

from . import build as _build

PRECISION_TF32 = 0
PRECISION_3XTF32 = 1

EXPORTED_SYMBOLS = (
    "triturus_b200_version",
    "triturus_b200_strerror",
    "triturus_b200_lm2exp_workspace_bytes",
    "triturus_b200_lm2exp_launches",
    "triturus_b200_lt2exp_launches",
    "triturus_b200_lt2exp_plan",
    "triturus_b200_lm2exp_plan",
    "triturus_b200_lm2exp_f32",
    "triturus_b200_lm2exp_chain_launches",
    "triturus_b200_lm2exp_chain_f32",
    "triturus_b200_lt2exp_f32",
    "triturus_b200_lt2exp_workspace_bytes",
    "triturus_b200_lt2exp_ws_f32",
    "triturus_b200_lt2exp_chain_f32",
    "triturus_b200_colmax_f32",
    "triturus_b200_selftest_wait_timeout",
    "triturus_b200_mm_f32",
    "triturus_b200_lm2exp_static_max_columns",
    "triturus_b200_lm2exp_f32_static",
)


class NativeLibraryError(RuntimeError):
    """The shared library is missing, cannot be loaded, or returned an error code."""


def _open() -> ctypes.CDLL:
    path = _build.LIB_PATH
    if _build.is_stale():
        # First use in a fresh checkout, or a source file is newer than the library: build in-tree (a no-op
        # when the library is fresh).  Without a compiler an existing library is used as it is; a missing one
        # is fatal by design.
        try:
            _build.build()
        except Exception as exc:  # noqa: BLE001
            if not path.exists():
                raise NativeLibraryError(
                    f"{path} is missing and could not be built ({exc}); run `python -m triturus_b200.build`"
                ) from exc
    try:
        return ctypes.CDLL(os.fspath(path))
    except OSError as exc:
        raise NativeLibraryError(f"cannot load {path}: {exc}") from exc


def _load() -> ctypes.CDLL:
    lib = _open()
    try:
        return _bind(lib)
    except AttributeError:
        # The library on disk predates a symbol this module binds (sources were updated): unload it,
        # rebuild once and load the new file.
        import _ctypes

        _ctypes.dlclose(lib._handle)
        del lib
        _build.build(force=True)
        return _bind(_open())


def _bind(lib: ctypes.CDLL) -> ctypes.CDLL:
    i64p = POINTER(c_int64)
    lib.triturus_b200_version.restype = c_int
    lib.triturus_b200_version.argtypes = []
    lib.triturus_b200_strerror.restype = c_char_p
    lib.triturus_b200_strerror.argtypes = [c_int]
    lib.triturus_b200_lm2exp_workspace_bytes.restype = c_size_t
    lib.triturus_b200_lm2exp_workspace_bytes.argtypes = [c_int64] * 4
    lib.triturus_b200_lm2exp_launches.restype = c_int
    lib.triturus_b200_lm2exp_launches.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int, c_int]
    lib.triturus_b200_lt2exp_launches.restype = c_int
    lib.triturus_b200_lt2exp_launches.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]
    lib.triturus_b200_lt2exp_plan.restype = c_int
    lib.triturus_b200_lt2exp_plan.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]
    lib.triturus_b200_lm2exp_plan.restype = c_int
    lib.triturus_b200_lm2exp_plan.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int, c_int]
    lib.triturus_b200_lm2exp_f32.restype = c_int
    lib.triturus_b200_lm2exp_f32.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, i64p, i64p, i64p,
        c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_lm2exp_chain_launches.restype = c_int
    lib.triturus_b200_lm2exp_chain_launches.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int]
    lib.triturus_b200_lm2exp_chain_f32.restype = c_int
    lib.triturus_b200_lm2exp_chain_f32.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, i64p, i64p, i64p,
        c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_lt2exp_f32.restype = c_int
    lib.triturus_b200_lt2exp_f32.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
        i64p, i64p, i64p, i64p, c_int, c_int, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_lt2exp_workspace_bytes.restype = c_size_t
    lib.triturus_b200_lt2exp_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]
    lib.triturus_b200_lt2exp_ws_f32.restype = c_int
    lib.triturus_b200_lt2exp_ws_f32.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
        i64p, i64p, i64p, i64p, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_lt2exp_chain_f32.restype = c_int
    lib.triturus_b200_lt2exp_chain_f32.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
        i64p, i64p, i64p, i64p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_lm2exp_static_max_columns.restype = c_size_t
    lib.triturus_b200_lm2exp_static_max_columns.argtypes = []
    lib.triturus_b200_lm2exp_f32_static.restype = c_int
    lib.triturus_b200_lm2exp_f32_static.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, i64p, i64p, i64p,
        c_int, c_int, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.triturus_b200_selftest_wait_timeout.restype = c_int
    lib.triturus_b200_selftest_wait_timeout.argtypes = [c_void_p, c_int64, c_void_p]
    lib.triturus_b200_mm_f32.restype = c_int
    lib.triturus_b200_mm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, i64p, i64p, i64p,
                                         c_int, c_void_p, c_void_p]  # fmt: skip
    lib.triturus_b200_colmax_f32.restype = c_int
    lib.triturus_b200_colmax_f32.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, i64p, c_void_p]
    return lib


LIB = _load()


def strerror(code: int) -> str:
    return LIB.triturus_b200_strerror(int(code)).decode()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}: {strerror(rc)}")


_I64x3 = c_int64 * 3
_I64x4 = c_int64 * 4


def _i64(vals) -> ctypes.Array:
    n = len(vals)
    return _I64x3(*vals) if n == 3 else _I64x4(*vals) if n == 4 else (c_int64 * n)(*vals)


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise NativeLibraryError(
                "triturus_b200 ops run only on CUDA tensors (sm_100a); there is no CPU implementation"
            )


# One zero-initialised status word per device, shared by all launches on it.  A kernel writes a positive
# code there only when one of its bounded waits gives up; `check_status` reads it back.
_STATUS = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATUS.get(idx)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = st
    return st


_LM_WORKSPACE: dict[tuple[int, int], torch.Tensor] = {}


def _lm2exp_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """The lm2exp workspace of the current stream of `device`: kept between calls and created zero-filled, so
    that the flag words at its start (the optimistic stabiliser's) are down unless a call on this stream left
    them up - a fresh allocation per call would put them on whatever the block held before.  Grows by doubling;
    calls on one stream are ordered, calls on different streams get different buffers."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, int(_raw_stream(idx)))
    ws = _LM_WORKSPACE.get(key)
    if ws is None or ws.numel() * 4 < nbytes:
        n = max(nbytes, 1 << 16, 0 if ws is None else 2 * ws.numel() * 4)
        ws = torch.zeros((n + 3) // 4, dtype=torch.float32, device=torch.device("cuda", idx))
        _LM_WORKSPACE[key] = ws
    return ws


def check_status(device=None) -> None:
    """Synchronise `device` and raise if any kernel launched through this module reported a time-out."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    elif isinstance(device, int):
        device = torch.device("cuda", device)
    st = _status_word(device)
    code = int(st.item())
    if code != 0:
        st.zero_()
        raise NativeLibraryError(f"device-side failure {code}: {strerror(code)}")


def _tma_ok(t: torch.Tensor) -> bool:
    """Innermost stride 1, other strides positive multiples of 4 elements, base 16-byte aligned: what a TMA
    tensor map needs."""
    if t.data_ptr() % 16 != 0 or not (t.shape[-1] == 1 or t.stride(-1) == 1):
        return False
    return all(t.shape[d] == 1 or (t.stride(d) > 0 and t.stride(d) % 4 == 0) for d in range(t.dim() - 1))


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Return `t` or a padded copy that meets `_tma_ok`.  The logical shape is unchanged."""
    if _tma_ok(t):
        return t
    inner = t.shape[-1]
    padded = (inner + 3) // 4 * 4
    buf = torch.empty(*t.shape[:-1], padded, dtype=t.dtype, device=t.device)
    view = buf[..., :inner]
    view.copy_(t)
    return view


# Problems up to this many FLOP take operands that break the tensor-map rules in place (the single-CTA kernel then
# fetches them element by element, ~3x slower per k-block than through TMA); larger ones get the padded copy, which
# is the cheaper of the two there.  Measured: R24 150x101x203 0.035 ms in place / 0.072 ms with the copy;
# R32 1024x1024x1022 0.75 / 0.26 ms; R128 256x256x8190 1.20 / 1.60 ms in TF32 but 2.97 / 2.32 ms in 3xTF32.
_IN_PLACE_MAX_FLOP = 8e9


def _in_place_small(t: torch.Tensor, flop: float, variant: int, want_colmax: bool) -> bool:
    """True when `t` should go to the library as it is although a tensor map cannot describe it."""
    tile = int(variant) % 100000
    return (flop <= _IN_PLACE_MAX_FLOP and not want_colmax and tile in _SINGLE_CTA_TILES
            and t.dtype == torch.float32 and t.data_ptr() % 4 == 0)


def _lm2exp_a_operand(a: torch.Tensor, K: int) -> torch.Tensor:
    """`a` [R,I,J] as the library takes it: unchanged when j is contiguous and the TMA rules hold; a
    transposed view (i contiguous, the other strides multiples of 4 elements, base 16-byte aligned) can be
    read in place as an MN-major tensor-core operand; otherwise a padded copy.

    Reading the view in place makes the contraction kernel about 16 % slower (four TMA boxes per tile and the
    MN-major operand fetch; measured 13 % on R32 x 1024^3, 18 % on R128 I=J=256 K=8192), a transposing copy
    runs at about 0.9 TB/s of `a`: the cheaper of the two is taken from a rough estimate of the kernel time."""
    R, I, J = a.shape
    if J > 1 and a.stride(2) != 1 and (I == 1 or a.stride(1) == 1) and a.data_ptr() % 16 == 0:
        if a.stride(2) > 0 and a.stride(2) % 4 == 0 and (R == 1 or (a.stride(0) > 0 and a.stride(0) % 4 == 0)):
            kernel_s = max(2.0 * R * I * J * K / 4e14, 4.0 * R * (I * J + J * K + I * K) / 4e12)
            copy_s = 4.0 * R * I * J / 0.9e12 + 5e-6
            if copy_s > 0.16 * kernel_s:
                return a
    return _tma_ready(a)


_SINGLE_CTA_TILES = (0, 1281, 1282, 2561, 2562)


def _lm2exp_b_operand(b: torch.Tensor, variant: int, flop: float = float("inf"), want_colmax: bool = False) -> torch.Tensor:
    """b as the kernel takes it.  Unchanged when the TMA rules hold.  A transposed view (j contiguous, e.g.
    `x.transpose(1, 2)` of a contiguous x) that meets them otherwise is read in place as a K-major operand by the
    single-CTA kernel, with the pre-pass stabiliser; variant codes that ask for a pair tile or the fused max pass
    get a copy instead.  Anything else goes in place when the problem is small (`_in_place_small`), else as a
    padded copy."""
    R, J, K = b.shape
    tile, stab = int(variant) % 100000, int(variant) // 100000
    if _tma_ok(b):
        return b
    if K > 1 and b.stride(2) != 1 and (J == 1 or b.stride(1) == 1) and b.data_ptr() % 16 == 0:
        if b.stride(2) > 0 and b.stride(2) % 4 == 0 and (R == 1 or (b.stride(0) > 0 and b.stride(0) % 4 == 0)):
            return b if (tile in _SINGLE_CTA_TILES and stab < 2) else _tma_ready(b)
    if _in_place_small(b, flop, variant, want_colmax):
        return b
    return _tma_ready(b)


def colmax(x: torch.Tensor) -> torch.Tensor:
    """Clamped column maximum of x[R, J, K] over J -> [R, K] (the stabiliser pre-pass)."""
    _require_cuda(x)
    R, J, K = x.shape  # (any strides: the kernel reads 16 bytes at a time where they allow it, else 4)
    m = torch.empty((R, K), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = LIB.triturus_b200_colmax_f32(x.data_ptr(), m.data_ptr(), R, J, K, _i64(x.stride()), stream)
    _check(rc, "triturus_b200_colmax_f32")
    return m


class _on_device:
    """Make `device` current for the duration of a launch; free when it already is (the common case)."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self) -> int:
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self.idx

    def __exit__(self, *exc) -> None:
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)


_raw_stream = torch._C._cuda_getCurrentRawStream  # cudaStream_t of torch's current stream, as an int


def _lm2exp_impl(a: torch.Tensor, b: torch.Tensor, precision: int, variant: int) -> torch.Tensor:
    _require_cuda(a, b)
    R, I, J = a.shape
    K = b.shape[2]
    flop = 2.0 * R * I * J * K
    a = a if _in_place_small(a, flop, variant, False) else _lm2exp_a_operand(a, K)
    b = _lm2exp_b_operand(b, variant, flop, False)
    out = torch.empty((R, I, K), dtype=torch.float32, device=a.device)
    ws_bytes = int(LIB.triturus_b200_lm2exp_workspace_bytes(R, I, J, K))
    with _on_device(a.device) as idx:
        ws = _lm2exp_workspace(a.device, ws_bytes)
        rc = LIB.triturus_b200_lm2exp_f32(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), R, I, J, K,
            _i64(a.stride()), _i64(b.stride()), _i64(out.stride()),
            int(precision), int(variant), ws.data_ptr(), ws_bytes,
            _status_word(a.device).data_ptr(), _raw_stream(idx),
        )  # fmt: skip
    _check(rc, "triturus_b200_lm2exp_f32")
    return out


def _lm2exp_chain_impl(
    a: torch.Tensor, b: torch.Tensor, b_colmax: torch.Tensor | None, want_colmax: bool, precision: int, variant: int
) -> tuple[torch.Tensor, torch.Tensor]:
    """lm2exp as a link of a chain: takes the column maxima of b when the caller has them and can return
    those of the result.  Returns (out, out_colmax); out_colmax is an empty tensor when not requested."""
    _require_cuda(a, b)
    R, I, J = a.shape
    K = b.shape[2]
    flop = 2.0 * R * I * J * K
    a = a if _in_place_small(a, flop, variant, want_colmax) else _lm2exp_a_operand(a, K)
    b = _lm2exp_b_operand(b, variant, flop, want_colmax)
    out = torch.empty((R, I, K), dtype=torch.float32, device=a.device)
    out_colmax = torch.empty((R, K) if want_colmax else (0,), dtype=torch.float32, device=a.device)
    if b_colmax is not None:
        _require_cuda(b_colmax)
        if b_colmax.shape != (R, K) or b_colmax.dtype != torch.float32 or b_colmax.device != b.device:
            raise ValueError(f"b_colmax must be a float32 [{R}, {K}] tensor on {b.device}")
        b_colmax = b_colmax.contiguous()
        ws_ptr, ws_bytes, ws = None, 0, None
    else:
        ws_bytes = int(LIB.triturus_b200_lm2exp_workspace_bytes(R, I, J, K))
        with _on_device(a.device):
            ws = _lm2exp_workspace(a.device, ws_bytes)
        ws_ptr = ws.data_ptr()
    with _on_device(a.device) as idx:
        rc = LIB.triturus_b200_lm2exp_chain_f32(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), R, I, J, K,
            _i64(a.stride()), _i64(b.stride()), _i64(out.stride()),
            int(precision), int(variant),
            b_colmax.data_ptr() if b_colmax is not None else None,
            out_colmax.data_ptr() if want_colmax else None,
            ws_ptr, ws_bytes, _status_word(a.device).data_ptr(), _raw_stream(idx),
        )  # fmt: skip
    _check(rc, "triturus_b200_lm2exp_chain_f32")
    return out, out_colmax


def _lt2exp_impl(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, precision: int, variant: int) -> torch.Tensor:
    _require_cuda(w, a, b)
    R, S, I, J = w.shape
    K = a.shape[2]
    w = _tma_ready(w)
    # a and b are read with ordinary loads and go in as they are, whatever their strides (16-byte loads when they
    # allow it; a view with a k stride other than 1 is read 4 bytes at a time, uncoalesced but without a copy)
    out = torch.empty((R, S, K), dtype=torch.float32, device=a.device)
    with _on_device(a.device) as idx:
        # scratch memory for tiles that several CTAs share (the end-to-end form of the contraction split)
        ws_bytes = int(LIB.triturus_b200_lt2exp_workspace_bytes(R, S, I, J, K, int(precision), int(variant)))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device) if ws_bytes else None
        rc = LIB.triturus_b200_lt2exp_ws_f32(
            w.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), R, S, I, J, K,
            _i64(w.stride()), _i64(a.stride()), _i64(b.stride()), _i64(out.stride()),
            int(precision), int(variant), ws.data_ptr() if ws is not None else None, ws_bytes,
            _status_word(a.device).data_ptr(), _raw_stream(idx),
        )  # fmt: skip
    _check(rc, "triturus_b200_lt2exp_ws_f32")
    return out


def mm_impl(a: torch.Tensor, b: torch.Tensor, precision: int) -> torch.Tensor:
    """out = a @ b for 2-D fp32 CUDA tensors through the contraction pipeline (the reference's triturus/mm.py)."""
    _require_cuda(a, b)
    a = _tma_ready(a)
    b = _tma_ready(b)
    M, K = a.shape
    N = b.shape[1]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    with _on_device(a.device) as idx:
        rc = LIB.triturus_b200_mm_f32(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, K, N,
            (c_int64 * 2)(*a.stride()), (c_int64 * 2)(*b.stride()), (c_int64 * 2)(*out.stride()),
            int(precision), _status_word(a.device).data_ptr(), _raw_stream(idx),
        )  # fmt: skip
    _check(rc, "triturus_b200_mm_f32")
    return out


def _colmax_arg(t: torch.Tensor | None, R: int, K: int, like: torch.Tensor, name: str) -> torch.Tensor | None:
    if t is None:
        return None
    _require_cuda(t)
    if t.shape != (R, K) or t.dtype != torch.float32 or t.device != like.device:
        raise ValueError(f"{name} must be a float32 [{R}, {K}] tensor on {like.device}")
    return t.contiguous()


def _lt2exp_chain_impl(
    w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, a_colmax: torch.Tensor | None,
    b_colmax: torch.Tensor | None, want_colmax: bool, precision: int, variant: int,
) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """lt2exp as a link of a chain: takes the column maxima of a and b when the caller has them and can
    return those of the result.  Returns (out, out_colmax); out_colmax is empty when not requested."""
    _require_cuda(w, a, b)
    R, S, I, J = w.shape
    K = a.shape[2]
    w = _tma_ready(w)
    a_colmax = _colmax_arg(a_colmax, R, K, a, "a_colmax")
    b_colmax = _colmax_arg(b_colmax, R, K, a, "b_colmax")
    out = torch.empty((R, S, K), dtype=torch.float32, device=a.device)
    out_colmax = torch.empty((R, K) if want_colmax else (0,), dtype=torch.float32, device=a.device)
    with _on_device(a.device) as idx:
        rc = LIB.triturus_b200_lt2exp_chain_f32(
            w.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), R, S, I, J, K,
            _i64(w.stride()), _i64(a.stride()), _i64(b.stride()), _i64(out.stride()),
            int(precision), int(variant),
            a_colmax.data_ptr() if a_colmax is not None else None,
            b_colmax.data_ptr() if b_colmax is not None else None,
            out_colmax.data_ptr() if want_colmax else None,
            _status_word(a.device).data_ptr(), _raw_stream(idx),
        )  # fmt: skip
    _check(rc, "triturus_b200_lt2exp_chain_f32")
    return out, out_colmax


# ---------------------------------------------------------------------------- torch custom ops
# torch.ops.triturus.lm2exp / torch.ops.triturus.lt2exp: CUDA only, with shape-inferring fake kernels so
# the ops trace under torch.compile / FakeTensor.  The reference defines no autograd for these ops.

lm2exp_op = torch.library.custom_op("triturus::lm2exp", _lm2exp_impl, mutates_args=(), device_types="cuda")
lt2exp_op = torch.library.custom_op("triturus::lt2exp", _lt2exp_impl, mutates_args=(), device_types="cuda")
lm2exp_chain_op = torch.library.custom_op(
    "triturus::lm2exp_chain", _lm2exp_chain_impl, mutates_args=(), device_types="cuda"
)


def lm2exp_call(a: torch.Tensor, b: torch.Tensor, precision: int, variant: int) -> torch.Tensor:
    """Eager calls go straight to the C ABI (the dispatcher round trip of a Python custom op costs more than
    the kernel of a small problem); under torch.compile the registered op is what gets traced."""
    if torch.compiler.is_compiling():
        return lm2exp_op(a, b, precision, variant)
    return _lm2exp_impl(a, b, precision, variant)


def lm2exp_chain_call(a, b, b_colmax, want_colmax: bool, precision: int, variant: int):
    if torch.compiler.is_compiling():
        return lm2exp_chain_op(a, b, b_colmax, want_colmax, precision, variant)
    return _lm2exp_chain_impl(a, b, b_colmax, want_colmax, precision, variant)


lt2exp_chain_op = torch.library.custom_op(
    "triturus::lt2exp_chain", _lt2exp_chain_impl, mutates_args=(), device_types="cuda"
)


def lt2exp_chain_call(w, a, b, a_colmax, b_colmax, want_colmax: bool, precision: int, variant: int):
    if torch.compiler.is_compiling():
        return lt2exp_chain_op(w, a, b, a_colmax, b_colmax, want_colmax, precision, variant)
    return _lt2exp_chain_impl(w, a, b, a_colmax, b_colmax, want_colmax, precision, variant)


@lt2exp_chain_op.register_fake
def _lt2exp_chain_fake(w, a, b, a_colmax, b_colmax, want_colmax, precision, variant):
    out = a.new_empty((w.shape[0], w.shape[1], a.shape[2]))
    return out, a.new_empty((w.shape[0], a.shape[2]) if want_colmax else (0,))


def lt2exp_call(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, precision: int, variant: int) -> torch.Tensor:
    if torch.compiler.is_compiling():
        return lt2exp_op(w, a, b, precision, variant)
    return _lt2exp_impl(w, a, b, precision, variant)


@lm2exp_op.register_fake
def _lm2exp_fake(a, b, precision, variant):
    return a.new_empty((a.shape[0], a.shape[1], b.shape[2]))


@lm2exp_chain_op.register_fake
def _lm2exp_chain_fake(a, b, b_colmax, want_colmax, precision, variant):
    out = a.new_empty((a.shape[0], a.shape[1], b.shape[2]))
    return out, a.new_empty((a.shape[0], b.shape[2]) if want_colmax else (0,))


@lt2exp_op.register_fake
def _lt2exp_fake(w, a, b, precision, variant):
    return a.new_empty((w.shape[0], w.shape[1], a.shape[2]))
