"""The kernel interface of the engine: thin, checked Python wrappers around the
``extern "C"`` entry points of the CUDA library.

Every operation writes into tensors the caller owns (nothing is allocated here),
runs on the current CUDA stream and raises :class:`KernelError` for a size or
type a kernel does not take.  There is no fallback: if the library cannot be
built or loaded, constructing :class:`CudaOps` fails.

``tests/plain_ops.py`` holds a plain PyTorch twin of each operation with the same
signature; the kernel tests compare the two.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass

import torch

from . import build as _build

ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2, "relu2": 3, "silu": 4}
# activations with learned numbers (how many): applied by ``learned_act`` between two linears
LEARNED_ACTIVATIONS = {"xielu": 2}
_LEARNED_CODES = {"xielu": 5}


def learned_constants(act: str, values) -> tuple[float, float]:
    """The two numbers a kernel takes for an activation with learned numbers.  xielu, values
    (p, q): softplus(p) and 1/2 + softplus(q), formed in double."""
    if act != "xielu" or len(values) != LEARNED_ACTIVATIONS["xielu"]:
        raise KernelError(f"activation {act!r} with {len(values)} numbers not taken")
    sp = lambda v: math.log1p(math.exp(-abs(v))) + max(v, 0.0)      # softplus
    return sp(values[0]), 0.5 + sp(values[1])
EXPERT_ACTIVATIONS = {"clamped": 0, "silu": 1, "relu2": 2}
_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


@dataclass(frozen=True)
class AttentionGeometry:
    """Sizes an attention layer hands to the cache and attention kernels."""

    n_heads: int
    n_kv_heads: int
    head_dim: int
    page_size: int
    num_pages: int
    max_pages: int          # row length of the block table
    q_off: int              # column of q / k / v in a row of the fused projection
    k_off: int
    v_off: int
    qkv_stride: int
    window: int = 0         # 0: every earlier key; w: the last w keys

    def page_elems(self) -> int:
        return 2 * self.n_kv_heads * self.page_size * self.head_dim


@dataclass
class AttentionPlan:
    """Work lists of one step for the specialised attention kernels, in device memory.

    ``data`` (int32): ``[0]`` number of single-query tokens, ``[1]`` number of 128-query
    tiles, ``[2]`` longest context among the single-query tokens, ``[3]`` unused; then per
    single-query token (``n_rows`` slots) its flat index, request row and position; then per
    tile (``tile_slots`` slots) the flat index of its first query, its number of queries, its
    request row and the position of its first query.
    ``decode_cap`` / ``tile_cap`` are the grid sizes the kernels are launched with (at
    least the counts; fixed per size class so that a captured graph stays valid)."""

    data: torch.Tensor
    n_rows: int
    decode_cap: int
    tile_cap: int
    single_new: bool = False     # every single-query token is the only new token of its request

    @property
    def tile_slots(self) -> int:
        return plan_tile_slots(self.n_rows)


def pack_weight_units(w: torch.Tensor) -> torch.Tensor:
    """A [features, k] bfloat16 matrix (k contiguous, k a multiple of 64) in the layout the
    persistent decode kernel streams: features padded with zero rows to a multiple of 16; tile j
    (rows 16 j .. 16 j + 15) is k / 64 boxes of [16 rows x 64 k] one behind the other, so that
    any run of boxes of a tile is contiguous; inside a box the 16-byte piece c of row r lies at
    piece c ^ (r & 7) of the row (the 128-byte XOR swizzle)."""
    n, k = w.shape
    if k % 64:
        raise KernelError(f"pack_weight_units: k = {k} is not a multiple of 64")
    n16 = -(-n // 16) * 16
    if n16 != n:
        w = torch.cat([w, w.new_zeros(n16 - n, k)])
    t = w.contiguous().view(n16 // 16, 16, k // 64, 8, 8)      # tile, row, box, piece, element
    out = torch.empty_like(t)
    for r in range(16):
        perm = [c ^ (r & 7) for c in range(8)]
        out[:, r] = t[:, r][:, :, perm]
    return out.permute(0, 2, 1, 3, 4).contiguous().view(-1)


@dataclass
class FusedTables:
    """Device records of a model for the persistent decode kernel (see ``fused_decode_build``)."""

    data: torch.Tensor            # uint8 on the device: layer records, then head and cache maps
    n_layers: int
    layer_bytes: int
    keep: list                    # the tensors the records point at

    @property
    def layers_ptr(self) -> int:
        return self.data.data_ptr()

    @property
    def tables_ptr(self) -> int:
        return self.data.data_ptr() + self.n_layers * self.layer_bytes


DECODE_MAX_NEW = 4        # requests bringing at most this many tokens use the decode kernel
PREFILL_TILE = 128


def _pow2(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


def size_class(n: int) -> int:
    """The size a count is rounded up to where shapes must repeat (captured graphs): powers of
    two up to 8, then four classes per doubling (10, 12, 14, 16, 20, 24, 28, 32, 40, 48, ...),
    so that padding stays below a quarter of the work."""
    if n <= 8:
        return _pow2(n)
    step = _pow2(n) // 8
    return -(-n // step) * step


def plan_tile_slots(n_rows: int) -> int:
    """Tile entries a plan holds: every tile a batch of n_rows tokens can have, rounded up to
    a power of two (grids are sized in powers of two when steps are captured)."""
    return _pow2(n_rows // PREFILL_TILE + n_rows // (DECODE_MAX_NEW + 1) + 1)


def plan_decode_ints(n_rows: int) -> int:
    """Ints of the single-query section: 3 per token, padded so that the tile section that
    follows is 16-byte aligned."""
    return (3 * n_rows + 3) // 4 * 4


_ERRORS = {-1: "unsupported size, type or option", -2: "bad argument"}

_lib = None


def load_library():
    """Build if needed and open the CUDA library (once per process)."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None
        _declare(_lib)
    return _lib


def _declare(lib) -> None:
    P, I, F = c_void_p, c_int, c_float
    sig = {
        "hs_embed": [P, P, P, P, P, P, I, I, I, I, I, P, I, F, P, P],
        "hs_layernorm": [P, P, P, P, P, I, I, F, I, P],
        "hs_linear_simt": [P, P, P, P, P, I, I, I, I, F, F, I, I, P],
        "hs_linear_tcgen05": [P, P, P, P, P, I, I, I, I, F, F, I, I, I, P, P, P, P],
        "hs_linear_tcgen05_scratch": [I, I, I, I, I, P, P],
        "hs_linear_skinny": [P, P, P, P, P, F, P, P, P, I, I, I, I, F, F, I, P, P, I, P],
        "hs_linear_skinny_scratch": [I, I, I, I, P, P],
        "hs_linear_skinny_argmax": [P, P, P, I, I, I, P, P, P, P, P, P, P, I, P],
        "hs_linear_skinny_argmax_scratch": [I, I, I, P],
        "hs_kv_append": [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "hs_attention_simt": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, I, P, P],
        "hs_attention_simt_grouped": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, I, I,
                                      P, P],
        "hs_attention_decode_append": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I,
                                       F, I, I, I, I, P, P, P, P, P],
        "hs_attention_decode_mma": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, I, I, I,
                                    P, P, P, P, P],
        "hs_attention_prefill": [P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, F, P, P],
        "hs_attention_prefill_tc": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, I, F, P, P],
        "hs_argmax": [P, P, I, I, P],
        "hs_dyt_norm": [P, P, P, P, P, I, I, F, I, P],
        "hs_scale": [P, ctypes.c_longlong, F, P],
        "hs_rotary_pairs": [P, P, P, P, I, I, I, I, I, I, P],
        "hs_grouped_linear": [P, P, P, I, I, I, I, I, I, I, I, I, P],
        "hs_grouped_linear_mma": [P, P, P, I, I, I, I, I, I, I, I, I, P],
        "hs_latent_append": [P, P, P, P, P, P, I, I, I, I, I, F, I, I, I, I, P, P, I, P],
        "hs_latent_attention": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, I, P, I,
                                P, P, I, P, P],
        "hs_latent_prefill_mma": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, P, P,
                                  I, P],
        "hs_delta_prepare": [P] * 15 + [I] * 9 + [P, P],
        "hs_delta_recurrence": [P] * 10 + [I] * 8 + [P],
        "hs_delta_finish": [P, P, P, P, P, P, I, F, I, I, I, I, I, I, I, I, P, P],
        "hs_moe_route": [P, P, P, P, P, I, I, I, I, I, I, I, P, P],
        "hs_moe_experts": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P, P],
        "hs_moe_route_top": [P, P, P, P, P, P, I, I, I, I, I, P, P],
        "hs_rms_norm": [P, P, P, P, I, I, F, I, P, I, I, I, P],
        "hs_rms_norm_add": [P, P, P, P, P, P, F, P, I, I, F, F, I, P, P, F, P],
        "hs_cast_rows": [P, P, ctypes.c_longlong, P],
        "hs_gated_act": [P, P, P, P, P, I, I, I, I, I, P],
        "hs_qk_prepare": [P, P, P, P, P, P, P, P, I, I, I, I, I, F, I, I, I, I, I, I, I, I, P, P],
        "hs_biased_attention": [P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, I, F, F, I, I,
                                I, P, P, P, P],
        "hs_biased_attention_prefill": [P, P, P, P, P, P, I, P, P, I, P, I, I, I, I, I, I, I, I,
                                        F, F, I, I, P, P],
        "hs_lightning_recurrence": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, P, P, I,
                                    F, P],
        "hs_token_shift_mix": [P, P, P, P, I, I, P, P, P, P, I, I, I, I, P],
        "hs_timemix_decay": [P, P, P, P, I, I, I, P],
        "hs_timemix_recurrence": [P, P, I, P, P, P, P, P, P, P, P, I, I, I, I, P],
        "hs_head_norm_gate": [P, P, P, P, I, I, I, I, I, F, I, F, I, P],
        "hs_gather_mul": [P, P, P, I, I, P, P, P, I, I, I, I, I, I, P, P],
        "hs_moe_route_table": [P, P, P, I, P, P, P, I, I, I, I, P, P],
        "hs_span_prepare": [P, P, P, I, I, I, I, P, I, I, P, P, I, I, I, I, I, I, F, I, I, I, P, P],
        "hs_span_attention": [P, P, P, P, I, I, P, P, P, P, I, I, F, I, I, I, I, I, I, I, F, I, I,
                              I, P, P, P, P],
        "hs_span_attention_prefill": [P, P, P, P, I, I, P, P, I, P, P, P, I, I, F, I, I, I, I, I, I,
                                      F, I, P, P],
        "hs_layernorm_add": [P, P, P, P, F, P, P, P, F, I, I, I, P],
        "hs_learned_act_xielu": [P, P, ctypes.c_longlong, F, F, I, P],
        "hs_scale_softcap": [P, ctypes.c_longlong, F, F, P],
        "hs_rglru_conv": [P, P, I, I, P, P, P, I, P, P, P, I, I, I, P],
        "hs_rglru_scan": [P, P, I, P, P, P, I, I, I, P, P, P, P, P, I, I, I, I, F, I, P],
        "hs_rglru_step": [P, P, I, P, I, I, I, P, P, P, P, P, P, P, I, I, I, I, F, I, P],
        "hs_pooled_prepare": [P, P, P, I, P, P, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, I,
                              I, P, P, I, I, I, P, P],
        "hs_pooled_means": [P, P, I, I, P, P, I, I, P, P, I, I, I, I, I, I, P, P],
        "hs_pooled_attention": [P, P, P, P, I, I, P, P, I, I, P, P, P, I, I, I, I, I, I, I, F, I,
                                I, I, P, P, P, P],
        "hs_pooled_attention_prefill": [P, P, P, P, I, I, P, P, I, I, P, P, I, P, P, I, I, I, I,
                                        I, I, F, I, P, P],
        "hs_moe_sorted_scratch": [I, I, I, I, I, I, P, P],
        "hs_sample": [P, P, P, P, P, P, P, I, I, P, P, P, P],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    LL = ctypes.c_longlong
    lib.hs_decode_persistent_layer_bytes.restype = c_int
    lib.hs_decode_persistent_tables_bytes.restype = c_int
    lib.hs_decode_persistent_grid.restype = c_int
    lib.hs_decode_persistent_slices.argtypes = [I, I]
    lib.hs_decode_persistent_slices.restype = c_int
    lib.hs_decode_persistent_supports.argtypes = [I] * 7
    lib.hs_decode_persistent_supports.restype = c_int
    lib.hs_decode_persistent_layer.argtypes = [P] * 13 + [F, F, F, I, I, I, LL]
    lib.hs_decode_persistent_layer.restype = c_int
    lib.hs_decode_persistent_tables.argtypes = [P, P, I, I, P, LL]
    lib.hs_decode_persistent_tables.restype = c_int
    lib.hs_decode_persistent.argtypes = ([P, P, I, P, P, P, P, F] + [I] * 5 + [P, I, I]
                                         + [P] * 11 + [I] + [P] * 7 + [I] * 4 + [P, P, I, P])
    lib.hs_decode_persistent.restype = c_int
    lib.hs_set_pdl.argtypes = [I]
    lib.hs_set_pdl.restype = None
    lib.hs_set_split_clusters.argtypes = [I]
    lib.hs_set_split_clusters.restype = None


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _want(t, name, dtype=None, dim=None, cuda=True):
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if cuda and not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list, set)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name}: dtype {t.dtype} not accepted (want {dtype})")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name}: expected {dim} dimensions, got shape {tuple(t.shape)}")
    return t


_FLOATS = (torch.float32, torch.bfloat16)


class CudaOps:
    """The hand-written sm_100a kernels, one method per operation."""

    name = "cuda"

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise KernelError("hetero_serve_b200 needs a CUDA device: its kernels have no CPU path")
        dev = torch.device("cuda" if device is None else device)
        if dev.type != "cuda":
            raise KernelError(f"hetero_serve_b200 needs a CUDA device, got {dev}")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        # One object drives one device.  Its kernels are launched on that device's current
        # stream, so the device must be current while they are (the runner sees to it).
        self.device = dev
        self.lib = load_library()
        self.launches = 0          # kernels launched through this object (graph captures count once)
        self.tensor_cores = True   # bfloat16 linears on tcgen05 (False: CUDA cores, for tests)
        self.fast_attention = True  # bfloat16 attention on the split-context / tensor-core kernels
        self.tc_attention = True    # head size 64: prompt portions on the tcgen05 attention kernel
        self.sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        self.fuse_norm = True      # LayerNorm fused into the few-row linear kernel
        self.fuse_argmax = True    # greedy choice fused into the few-row head (linear_argmax)
        self.fuse_append = True    # key/value append fused into the decode attention
        self.pdl = True            # programmatic dependent launch (see the property below)
        self._skinny_need: dict = {}
        self._moe_need: dict = {}
        self.latent_mma = True      # prompt portions of latent attention on the tensor cores
        self.biased_mma = True      # prompt portions of the biased chunk attention likewise
        self.pooled_mma = True      # ... and of the attention over a window and pooled blocks
        self.span_mma = True        # ... and of the attention with a distance slope and a window
        self.folds_pooled_means = True   # pooled_prepare takes the companion pool (single tokens)
        self.lightning_bulk_rows = 64   # from this many tokens a step on, lightning attention
        #                                 activates its rows in a pass of their own
        self.latent_splits = None   # blocks a token's keys are split over in latent attention
        #                             (None: chosen from the number of tokens in the step)
        self.sorted_experts = True  # many (token, expert) pairs in bfloat16: sorted by expert and
        #                             run as tiles on the tensor cores (False: a product per pair)
        self._tc_need: dict = {}
        self._scratch: dict = {}
        self._retired: list = []
        self.decode_force = None   # (wide code, slices) of the decode attention, for tuning
        self.decode_mma = True     # tensor-core decode attention where the shape allows it
        #                            (head size 32/64/128, at most 16 query heads per kv head)
        self.takes_status_word = True   # sample() can store the status word behind the tokens
        self.tile_n = 0            # 0: chosen per shape; 64/128/192/256 force a tile width
        self.cta_pairs = -1        # -1: pairs of CTAs (cta_group::2) when there are many rows;
        #                            0: never; 1: always
        self.split_clusters = True  # few rows split over k: the splits of a tile exchange their
        #                            shares inside a thread-block cluster (False: through scratch)
        self.fused_decode_on = False  # pure decode steps of up to 16 tokens as ONE persistent kernel
        #                             (measured slower than the layer-by-layer path: off)
        self.skinny_max_rows = 16  # up to this many rows the weight-streaming kernel is used
        #                            (measured: from 17 rows on the tcgen05 kernel's split over k wins)
        # pipeline time-outs of the TMA/tcgen05 kernels are ORed into this word; the runner
        # replaces it with its own so that they surface with the step's results
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # -- kernels that parts bring themselves -------------------------------------------
    def stream(self) -> int:
        """The raw CUDA stream (of this object's device) kernels are to be launched on."""
        return self._stream()

    def register_kernel(self, symbol: str, argtypes, lib=None):
        """Declare an ``extern "C"`` entry point (returning int in the convention of this
        library: 0, a negative HS_ERR_* code or a positive cudaError_t) and return a function
        that calls it, counts the launch and raises :class:`KernelError` on a non-zero code.
        ``lib`` is a library opened with :meth:`load_extension`; by default the package's
        own.  A part calls this once (in ``bind``) and the returned function in ``forward``
        with raw pointers (``tensor.data_ptr()``), sizes and ``ops.stream()``."""
        lib = lib or self.lib
        try:
            fn = getattr(lib, symbol)
        except AttributeError:
            raise KernelError(f"the library exports no symbol {symbol!r}") from None
        fn.argtypes = list(argtypes)
        fn.restype = c_int

        def call(*args):
            self.launches += 1
            _check(fn(*args), symbol)
        call.__name__ = symbol
        return call

    def load_extension(self, name: str, sources):
        """Build (once) and open a library of CUDA sources from outside the package; see
        :func:`hetero_serve_b200.kernels.build.build_extension`."""
        path = _build.build_extension(name, sources)
        try:
            return ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None

    @property
    def pdl(self) -> bool:
        """Programmatic dependent launch: kernels are launched so that their set-up (and what
        they fetch that no kernel of the step writes: weights, work lists) overlaps the end of
        the kernel before them; each waits before it first reads an earlier kernel's output.
        The few-row linear and the decode attention take it as an argument; the other kernels
        read a switch in the library, which is process-wide (the last setter wins)."""
        return self._pdl

    @pdl.setter
    def pdl(self, on: bool) -> None:
        self._pdl = bool(on)
        self.lib.hs_set_pdl(int(self._pdl))

    # -- embedding and norm -------------------------------------------------
    def embed(self, x, ids, pos, req, wte, wpe, status, feedback=None, scale=1.0):
        """x[t] = wte[ids[t]] * scale (+ wpe[pos[t]]); rows with req[t] < 0 become zero.  With
        ``feedback`` (int32 on the device) an id ``-(s + 1)`` stands for ``feedback[s]``."""
        _want(x, "x", torch.float32, 2)
        _want(wte, "wte", _FLOATS, 2)
        n, width = x.shape
        for t, nm in ((ids, "ids"), (pos, "pos"), (req, "req")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < n:
                raise KernelError(f"{nm}: {t.shape[0]} entries for {n} rows")
        if wte.shape[1] != width:
            raise KernelError(f"wte width {wte.shape[1]} != x width {width}")
        n_pos = 0
        if wpe is not None:
            _want(wpe, "wpe", wte.dtype, 2)
            if wpe.shape[1] != width:
                raise KernelError(f"wpe width {wpe.shape[1]} != x width {width}")
            n_pos = wpe.shape[0]
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
        self.launches += 1
        _check(self.lib.hs_embed(_ptr(x), _ptr(ids), _ptr(pos), _ptr(req), _ptr(wte), _ptr(wpe),
                                 n, width, wte.shape[0], n_pos, _DT[wte.dtype], _ptr(feedback),
                                 0 if feedback is None else feedback.shape[0], float(scale),
                                 _ptr(status), self._stream()), "embed")

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        """out[i] = LayerNorm(x[rows[i]] if rows is given else x[i]) * gamma + beta."""
        _want(out, "out", _FLOATS, 2)
        _want(x, "x", torch.float32, 2)
        _want(gamma, "gamma", torch.float32, 1)
        _want(beta, "beta", torch.float32, 1)
        n, width = out.shape
        if x.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
            raise KernelError("layernorm: widths of out, x, gamma, beta differ")
        if rows is not None:
            _want(rows, "rows", torch.int32, 1)
            if rows.shape[0] < n:
                raise KernelError("layernorm: fewer row indices than output rows")
        elif x.shape[0] < n:
            raise KernelError("layernorm: x has fewer rows than out")
        self.launches += 1
        _check(self.lib.hs_layernorm(_ptr(out), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(rows), n,
                                     width, float(eps), _DT[out.dtype], self._stream()),
               f"layernorm(width={width})")

    # -- linear ---------------------------------------------------------------
    def linear(self, out, a, w, bias=None, act="none", residual=None, act_values=()):
        """out = act(a @ w.T + bias) (+ residual).  a [M,K], w [N,K], out [M,N].  ``act`` is one
        of ACTIVATIONS, or of LEARNED_ACTIVATIONS with its learned numbers in ``act_values``
        (applied to the float32 sum, as ``learned_act`` does).

        ``residual`` is float32 [M,N] and may be ``out`` itself (accumulate in place)."""
        _want(a, "a", _FLOATS, 2)
        _want(w, "w", a.dtype, 2)
        _want(out, "out", _FLOATS, 2)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError(f"linear: shapes a{tuple(a.shape)} w{tuple(w.shape)} "
                              f"out{tuple(out.shape)} do not fit")
        if a.dtype == torch.float32 and out.dtype != torch.float32:
            raise KernelError("linear: float32 inputs give float32 outputs")
        if bias is not None:
            _want(bias, "bias", torch.float32, 1)
            if bias.shape[0] != N:
                raise KernelError("linear: bias length != N")
        if residual is not None:
            _want(residual, "residual", torch.float32, 2)
            if tuple(residual.shape) != (M, N):
                raise KernelError("linear: residual shape != out shape")
        if act in LEARNED_ACTIVATIONS:
            if len(act_values) != LEARNED_ACTIVATIONS[act]:
                raise KernelError(f"linear: activation {act!r} takes "
                                  f"{LEARNED_ACTIVATIONS[act]} numbers")
            code = (_LEARNED_CODES[act], *learned_constants(act, act_values))
        elif act in ACTIVATIONS:
            code = (ACTIVATIONS[act], 0.0, 0.0)
        else:
            raise KernelError(f"linear: unknown activation {act!r}")
        self._linear(out, a, w, bias, code, residual, M, N, K)

    def _linear(self, out, a, w, bias, act, residual, M, N, K):
        """``act`` is a code of ACTIVATIONS, or (code, a, b) with the two numbers of an
        activation that has some.  bfloat16 goes to the tcgen05 kernel when TMA can address the operands (K a multiple
        of 8, 16-byte aligned pointers); everything else, and all of float32, to the CUDA cores."""
        self.launches += 1
        act, act_a, act_b = act if isinstance(act, tuple) else (act, 0.0, 0.0)
        if a.dtype == torch.bfloat16 and self._skinny_ok(M, N, K):
            if self._skinny(out, a, None, w, bias, (act, act_a, act_b), residual, M, N, K):
                return
        if a.dtype == torch.bfloat16 and self.tensor_cores and K % 8 == 0:
            if CudaOps._lib_split_clusters != bool(self.split_clusters):   # a switch of the library
                CudaOps._lib_split_clusters = bool(self.split_clusters)
                self.lib.hs_set_split_clusters(int(CudaOps._lib_split_clusters))
            key = (M, N, K, self.tile_n, self.cta_pairs, bool(self.split_clusters))
            need = self._tc_need.get(key)
            if need is None:
                floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
                rc = self.lib.hs_linear_tcgen05_scratch(M, N, K, self.tile_n, self.cta_pairs,
                                                        ctypes.byref(floats),
                                                        ctypes.byref(counters))
                need = (floats.value, counters.value) if rc == 0 else (0, 0)
                self._tc_need[key] = need
            scratch = cnt = None
            if need[0]:
                scratch = self._scratch_buffer("tc_partial", need[0], torch.float32)
                cnt = self._scratch_buffer("tc_counters", need[1], torch.int32)
            code = self.lib.hs_linear_tcgen05(
                _ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), M, N, K, act,
                act_a, act_b, _DT[out.dtype], self.tile_n, self.cta_pairs, _ptr(scratch), _ptr(cnt),
                _ptr(self.status),
                self._stream())
            if code != -1:
                _check(code, f"linear_tcgen05(M={M},N={N},K={K})")
                return
        _check(self.lib.hs_linear_simt(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual),
                                       M, N, K, act, act_a, act_b, _DT[a.dtype],
                                       _DT[out.dtype], self._stream()),
               f"linear(M={M},N={N},K={K})")

    def _skinny_ok(self, M, N, K) -> bool:
        return self.tensor_cores and M <= self.skinny_max_rows

    def _skinny(self, out, a, norm, w, bias, act, residual, M, N, K) -> bool:
        """The weight-streaming kernel; ``norm = (x, gamma, beta, eps)`` fuses a LayerNorm of
        the float32 input.  False when the kernel does not take the shape."""
        key = (M, N, K, norm is not None)
        need = self._skinny_need.get(key)
        if need is None:
            floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
            code = self.lib.hs_linear_skinny_scratch(M, N, K, int(norm is not None),
                                                     ctypes.byref(floats), ctypes.byref(counters))
            need = (floats.value, counters.value) if code == 0 else False
            self._skinny_need[key] = need
        if need is False:
            return False
        scratch = cnt = None
        if need[0]:
            scratch = self._scratch_buffer("skinny_partial", need[0], torch.float32)
            cnt = self._scratch_buffer("skinny_counters", need[1], torch.int32)
        x = g = b = None
        eps = 0.0
        if norm is not None:
            x, g, b, eps = norm
        act, act_a, act_b = act if isinstance(act, tuple) else (act, 0.0, 0.0)
        code = self.lib.hs_linear_skinny(
            _ptr(out), _ptr(a), _ptr(x), _ptr(g), _ptr(b), float(eps), _ptr(w), _ptr(bias),
            _ptr(residual), M, N, K, act, act_a, act_b, _DT[out.dtype], _ptr(scratch), _ptr(cnt),
            int(self.pdl), self._stream())
        if code == -1:
            return False
        _check(code, f"linear_skinny(M={M},N={N},K={K})")
        return True

    def linear_argmax(self, out, a, w, tokens, feedback=None, feedback_slot=None,
                      status_word=None) -> bool:
        """out = a @ w.T as float32 logits AND tokens[m] = argmax of row m (lowest index on
        ties), in the one few-row kernel: its CTAs keep their best per row while they stream
        the table, the last to finish picks.  ``tokens`` has a word more than rows, which
        receives ``status_word``; ``feedback[feedback_slot[m]]`` gets row m's token as in
        `sample`.  False (nothing done) for shapes or types the kernel does not take: the
        caller then runs `linear` and `sample`."""
        if not (self.tensor_cores and self.fuse_argmax and a.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and out.dtype == torch.float32):
            return False
        _want(a, "a", torch.bfloat16, 2)
        _want(w, "w", torch.bfloat16, 2)
        _want(out, "out", torch.float32, 2)
        _want(tokens, "tokens", torch.int32, 1)
        M, K = a.shape
        N = w.shape[0]
        if M > self.skinny_max_rows or w.shape[1] != K or tuple(out.shape) != (M, N):
            return False
        if tokens.shape[0] < M + 1:
            raise KernelError("linear_argmax: tokens needs a word more than rows")
        if (feedback is None) != (feedback_slot is None):
            raise KernelError("linear_argmax: feedback and feedback_slot come together")
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
            _want(feedback_slot, "feedback_slot", torch.int32, 1)
            if feedback_slot.shape[0] < M:
                raise KernelError("linear_argmax: feedback_slot shorter than the rows")
        if status_word is not None:
            _want(status_word, "status_word", torch.int32, 1)
        key = ("argmax", M, N, K)
        need = self._skinny_need.get(key)
        if need is None:
            entries = ctypes.c_int(0)
            code = self.lib.hs_linear_skinny_argmax_scratch(M, N, K, ctypes.byref(entries))
            need = entries.value if code == 0 else False
            self._skinny_need[key] = need
        if need is False:
            return False
        val = self._scratch_buffer("argmax_val", need, torch.float32)
        idx = self._scratch_buffer("argmax_idx", need, torch.int32)
        cnt = self._scratch_buffer("argmax_counter", 1, torch.int32)
        code = self.lib.hs_linear_skinny_argmax(
            _ptr(out), _ptr(a), _ptr(w), M, N, K, _ptr(tokens), _ptr(feedback),
            _ptr(feedback_slot), _ptr(status_word), _ptr(val), _ptr(idx), _ptr(cnt),
            int(self.pdl), self._stream())
        if code == -1:
            return False
        _check(code, f"linear_argmax(M={M},N={N},K={K})")
        self.launches += 1
        return True

    def norm_linear(self, out, h, x, gamma, beta, eps, w, bias=None, act="none"):
        """out = act(LayerNorm(x) @ w.T + bias).  For few rows the normalisation is fused into
        the weight-streaming kernel; otherwise ``h`` receives LayerNorm(x) first."""
        M, K = x.shape
        N = w.shape[0]
        if (w.dtype == torch.bfloat16 and self.fuse_norm and self._skinny_ok(M, N, K)):
            _want(x, "x", torch.float32, 2)
            _want(w, "w", torch.bfloat16, 2)
            _want(out, "out", _FLOATS, 2)
            _want(gamma, "gamma", torch.float32, 1)
            _want(beta, "beta", torch.float32, 1)
            if w.shape[1] != K or tuple(out.shape) != (M, N) or gamma.shape[0] != K \
                    or beta.shape[0] != K:
                raise KernelError("norm_linear: shapes do not fit")
            if bias is not None:
                _want(bias, "bias", torch.float32, 1)
            if act not in ACTIVATIONS:
                raise KernelError(f"norm_linear: unknown activation {act!r}")
            self.launches += 1
            if self._skinny(out, None, (x, gamma, beta, eps), w, bias, ACTIVATIONS[act], None,
                            M, N, K):
                return
            self.launches -= 1
        self.layernorm(h, x, gamma, beta, eps)
        self.linear(out, h, w, bias, act=act)

    # -- cache and attention ------------------------------------------------------
    def _attn_common(self, qkv, pool, table, tok_pos, tok_req, g, n):
        _want(qkv, "qkv", _FLOATS, 2)
        _want(pool, "pool", qkv.dtype)
        _want(table, "table", torch.int32, 2)
        _want(tok_pos, "tok_pos", torch.int32, 1)
        _want(tok_req, "tok_req", torch.int32, 1)
        if qkv.shape[0] < n or tok_pos.shape[0] < n or tok_req.shape[0] < n:
            raise KernelError("attention: fewer rows than tokens")
        if qkv.shape[1] != g.qkv_stride or table.shape[1] != g.max_pages:
            raise KernelError("attention: geometry does not match the tensors")
        if pool.numel() != g.num_pages * g.page_elems():
            raise KernelError(f"attention: pool has {pool.numel()} elements, geometry wants "
                              f"{g.num_pages * g.page_elems()}")
        hd = g.head_dim
        if (g.q_off + g.n_heads * hd > g.qkv_stride or g.k_off + g.n_kv_heads * hd > g.qkv_stride
                or g.v_off + g.n_kv_heads * hd > g.qkv_stride):
            raise KernelError("attention: q/k/v columns exceed the fused row")

    def kv_append(self, pool, qkv, table, tok_pos, tok_req, g, status, n_tokens=None):
        """Write each token's key and value rows into its page (rows with req < 0 are skipped)."""
        n = qkv.shape[0] if n_tokens is None else n_tokens
        self._attn_common(qkv, pool, table, tok_pos, tok_req, g, n)
        self.launches += 1
        _check(self.lib.hs_kv_append(_ptr(pool), _ptr(qkv), _ptr(table), _ptr(tok_pos),
                                     _ptr(tok_req), n, g.n_heads, g.n_kv_heads, g.head_dim,
                                     g.page_size, g.num_pages, g.max_pages, g.q_off, g.k_off,
                                     g.v_off, g.qkv_stride, _DT[qkv.dtype], _ptr(status),
                                     self._stream()),
               f"kv_append(head_dim={g.head_dim})")

    def attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan=None,
                  _fuse_append=False):
        """out[t] = causal attention of token t's query over its request's pages.

        ``plan`` may carry a batch's work lists for the specialised kernels; the general
        kernel needs none."""
        _want(out, "out", qkv.dtype, 2)
        n = out.shape[0]
        if out.shape[1] != g.n_heads * g.head_dim:
            raise KernelError("attention: out width != n_heads * head_dim")
        self._attn_common(qkv, pool, table, tok_pos, tok_req, g, n)
        self._attention(out, qkv, pool, table, tok_pos, tok_req, g, float(scale), status, plan, n,
                        _fuse_append)

    # -- attention work lists ---------------------------------------------------------
    @staticmethod
    def attention_plan_ints(n_rows: int, n_requests: int) -> int:
        return 4 + plan_decode_ints(n_rows) + 4 * plan_tile_slots(n_rows)

    @staticmethod
    def plan_attention(view, host_batch, n_rows: int, n_requests: int, page_size: int,
                       bucketed: bool) -> tuple[int, int]:
        """Fill the plan section (a numpy int32 view of the step's metadata) for a batch given
        as ``[(request, slot, start, n_new)]`` in flat order; returns ``(decode_cap,
        tile_cap, single_new)``.  Requests bringing up to DECODE_MAX_NEW tokens go to the single-query
        list, the others are cut into tiles of 128 queries, longest context first."""
        dec = view[4:4 + 3 * n_rows]
        tiles = view[4 + plan_decode_ints(n_rows):]
        n_dec = n_tiles = max_ctx = 0
        t = 0
        single = True
        tile_list = []
        for row, (_req, _slot, start, n) in enumerate(host_batch):
            if n <= DECODE_MAX_NEW:
                single = single and n == 1
                for i in range(n):
                    dec[3 * n_dec:3 * n_dec + 3] = (t + i, row, start + i)
                    n_dec += 1
                max_ctx = max(max_ctx, start + n)
            else:
                for q0 in range(0, n, PREFILL_TILE):
                    tile_list.append((t + q0, min(PREFILL_TILE, n - q0), row, start + q0))
                    n_tiles += 1
            t += n
        # tiles with the most keys first, so that the long ones do not form the tail
        tile_list.sort(key=lambda ti: -(ti[3] + ti[1]))
        for i, ti in enumerate(tile_list):
            tiles[4 * i:4 * i + 4] = ti
        view[0], view[1], view[2], view[3] = n_dec, n_tiles, max_ctx, 0
        single = single and n_dec > 0
        if bucketed:
            return (size_class(n_dec) if n_dec else 0, size_class(n_tiles) if n_tiles else 0,
                    single)
        return n_dec, n_tiles, single

    def make_plan(self, host_batch, n_rows: int, page_size: int) -> AttentionPlan:
        """A plan built and uploaded on the spot (the runner packs it into the step's single
        upload instead)."""
        import numpy as np
        view = np.zeros(self.attention_plan_ints(n_rows, len(host_batch)), dtype=np.int32)
        dec, tiles, single = self.plan_attention(view, host_batch, n_rows, len(host_batch),
                                                 page_size, False)
        return AttentionPlan(torch.from_numpy(view).to(self.device), n_rows, dec, tiles, single)

    def _scratch_buffer(self, name, numel, dtype):
        key = (name, dtype)
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)       # captured graphs may still point into it
            buf = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self._scratch[key] = buf
        return buf

    def decode_wide(self, decode_cap: int, n_heads: int) -> int:
        """Warps per CTA of the decode attention: 16 (code 2) while token x head count is below
        the SM count, 8 (code 1) up to twice that, else 4 (code 0)."""
        if self.decode_force is not None:
            return self.decode_force[0]
        pairs = decode_cap * n_heads
        return 2 if pairs <= self.sm_count else (1 if pairs <= 2 * self.sm_count else 0)

    def decode_splits(self, decode_cap: int, n_heads: int, max_context: int) -> int:
        """Slices between CTAs the context of a single-query token is cut into: one wave of
        CTAs over the SMs, slices of at least 64 keys (in the manner of the reference's
        ``choose_num_splits``, heteroserve/model/paged_attn_v3.py:212-232).  Slices cost a
        round trip through scratch memory, so they are used only when token x head count is
        small."""
        pairs = max(1, decode_cap * n_heads)
        wide = self.decode_wide(decode_cap, n_heads)
        if self.decode_force is not None:
            return self.decode_force[1]
        want = max(1, round(self.sm_count / pairs)) if wide == 2 else 1
        per_warp = 32 * 16 * (4, 8, 16)[wide]        # keys a CTA can cover: 32 pages per warp
        need = -(-max_context // per_warp)
        return max(1, need, min(want, max(1, max_context // 64), 32))

    FAST_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
    _lib_split_clusters = True     # what the library's switch was last set to

    def _fast_ok(self, qkv, g, plan, n, scale=1.0) -> bool:
        return (plan is not None and self.fast_attention and qkv.dtype == torch.bfloat16
                and g.window == 0 and g.head_dim in self.FAST_HEAD_DIMS and plan.n_rows >= n
                and scale > 0)

    def attention_append(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status,
                         plan=None, writes=True):
        """Append the new keys/values to the pages (if ``writes``), then attention.  When the
        step is made of single decoded tokens only, the decode kernel does both in one launch."""
        n = out.shape[0]
        fuse = (writes and self.fuse_append and self._fast_ok(qkv, g, plan, n, scale)
                and plan.tile_cap == 0 and plan.decode_cap > 0 and plan.single_new)
        if writes and not fuse:
            self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
        self.attention(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                       _fuse_append=fuse)

    def _attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan, n,
                   fuse=False):
        if self._fast_ok(qkv, g, plan, n, scale):
            self._attention_fast(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                                 fuse)
            return
        self.launches += 1
        # steps of prompt portions (four tokens a request or more on average): a CTA serves four
        # neighbours of the batch, which share the staged keys when they are one request's
        # (with a work list: the step has prompt portions; the counts may be padded ones)
        group = 4 if (plan.tile_cap > 0 if plan is not None else n >= 4 * table.shape[0]) else 1
        _check(self.lib.hs_attention_simt_grouped(
            _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req), n,
            g.n_heads, g.n_kv_heads, g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off,
            g.k_off, g.v_off, g.qkv_stride, g.window, scale, _DT[qkv.dtype], group, _ptr(status),
            self._stream()), f"attention(head_dim={g.head_dim}, heads={g.n_heads})")

    def _attention_fast(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                        fuse=False):
        d = plan.data
        nr = plan.n_rows
        head = d
        dec_info = d[4:]
        tile_info = d[4 + plan_decode_ints(nr):]
        st = self._stream()
        if plan.decode_cap:
            max_ctx = g.max_pages * g.page_size
            group = g.n_heads // g.n_kv_heads
            use_mma = (self.decode_mma and self.decode_force is None
                       and g.head_dim in (32, 64, 128) and group <= 16)
            if use_mma:
                # slices of at most 2,048 keys; a long table and so few (token, head) pairs that
                # they leave SMs idle: more, shorter slices (of 512 keys or more), a CTA an SM
                splits = max(1, -(-max_ctx // 2048))
                pairs = plan.decode_cap * g.n_kv_heads
                if max_ctx >= 2048 and pairs * splits <= self.sm_count:
                    splits = max(splits, min(-(-max_ctx // 512), self.sm_count // pairs))
            else:
                splits = self.decode_splits(plan.decode_cap, g.n_heads, max_ctx)
            acc = ml = cnt = None
            if splits > 1:
                rows = plan.decode_cap * g.n_heads * splits
                acc = self._scratch_buffer("decode_acc", rows * g.head_dim, torch.float32)
                ml = self._scratch_buffer("decode_ml", rows * 2, torch.float32)
                cnt = self._scratch_buffer("decode_counters", plan.decode_cap * g.n_heads,
                                           torch.int32)
            self.launches += 1
            if use_mma:
                code = self.lib.hs_attention_decode_mma(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(dec_info), _ptr(head),
                    plan.decode_cap, g.n_heads, g.n_kv_heads, g.head_dim, g.page_size,
                    g.num_pages, g.max_pages, g.q_off, g.k_off, g.v_off, g.qkv_stride, scale,
                    splits, int(bool(fuse)), int(self.pdl), _ptr(acc), _ptr(ml), _ptr(cnt),
                    _ptr(status), st)
                what = f"attention_decode_mma(head_dim={g.head_dim})"
            else:
                code = self.lib.hs_attention_decode_append(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                    _ptr(dec_info), _ptr(head), plan.decode_cap, g.n_heads, g.n_kv_heads,
                    g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.k_off, g.v_off,
                    g.qkv_stride, g.window, scale, splits, int(bool(fuse)),
                    int(self.decode_wide(plan.decode_cap, g.n_heads)), int(self.pdl), _ptr(acc),
                    _ptr(ml), _ptr(cnt), _ptr(status), st)
                what = f"attention_decode(head_dim={g.head_dim})"
            if code == -1:
                # a shape the decode kernels do not take: the general kernel serves every token
                # of the batch (it needs no work list); a fused append is done first
                if fuse:
                    self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
                _check(self.lib.hs_attention_simt(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                    out.shape[0], g.n_heads, g.n_kv_heads, g.head_dim, g.page_size, g.num_pages,
                    g.max_pages, g.q_off, g.k_off, g.v_off, g.qkv_stride, g.window, scale,
                    _DT[qkv.dtype], _ptr(status), st),
                    f"attention(head_dim={g.head_dim}, heads={g.n_heads})")
                return
            _check(code, what)
        if plan.tile_cap:
            self.launches += 1
            counter = self._scratch_buffer("prefill_counter", 1, torch.int32)
            if self.tc_attention and g.head_dim == 64:
                code = self.lib.hs_attention_prefill_tc(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tile_info), _ptr(head),
                    plan.tile_cap, _ptr(counter), qkv.shape[0], g.n_heads, g.n_kv_heads,
                    g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.qkv_stride,
                    scale, _ptr(status), st)
                if code != -1:
                    _check(code, "attention_prefill_tc")
                    return
            _check(self.lib.hs_attention_prefill(
                _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                _ptr(tile_info), _ptr(head), plan.tile_cap,
                _ptr(self._scratch_buffer("prefill_counter", 1, torch.int32)), g.n_heads, g.n_kv_heads,
                g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.qkv_stride, scale,
                _ptr(status), st), f"attention_prefill(head_dim={g.head_dim})")

    # -- the whole decode step in one kernel ----------------------------------------
    FUSED_MAX_TOKENS = 16

    def fused_decode_supports(self, *, width, inner, n_heads, head_dim, n_kv_heads, page_size,
                              window) -> bool:
        """Whether the persistent decode kernel serves a model of these sizes at all (bfloat16,
        heads of 64 without grouping, pages of 16, widths in multiples of 64 up to 2,048)."""
        return bool(self.fused_decode_on and self.lib.hs_decode_persistent_supports(
            int(width), int(inner), int(n_heads), int(head_dim), int(n_kv_heads),
            int(page_size), int(window)))

    def fused_decode_build(self, layers, *, head_weight, pool, width, inner, vocab):
        """Descriptor records of a model for :meth:`fused_decode`: per layer call its four
        matrices (repacked here, see :func:`pack_weight_units`: the kernel keeps its own copy of
        every matrix, laid out so that what a CTA streams is contiguous), its vectors and
        constants, and once the head and the tensor map of the cache storage.  ``layers`` is a list of dictionaries with the keys ``w_qkv w_out
        w_fc w_mlp`` ([features, k] bfloat16), ``b_qkv b_out b_fc b_mlp ln1_g ln1_b ln2_g ln2_b``
        (float32 or None for the biases), ``eps1 eps2 scale act entry``; ``pool`` is the cache
        group's storage ``[entries, pages, 2, heads, 16, 64]``."""
        lib = self.lib
        lb, tb = lib.hs_decode_persistent_layer_bytes(), lib.hs_decode_persistent_tables_bytes()
        host = torch.zeros(len(layers) * lb + tb, dtype=torch.uint8)
        base = host.data_ptr()
        _want(pool, "pool", torch.bfloat16, 6)
        rows_per_entry = pool.shape[1] * pool.shape[2] * pool.shape[3] * pool.shape[4]
        keep = [pool]
        packs: dict[int, torch.Tensor] = {}
        for i, L in enumerate(layers):
            for nm in ("w_qkv", "w_out", "w_fc", "w_mlp"):
                _want(L[nm], nm, torch.bfloat16, 2)
            for nm in ("ln1_g", "ln1_b", "ln2_g", "ln2_b"):
                _want(L[nm], nm, torch.float32, 1)
            for nm in ("b_qkv", "b_out", "b_fc", "b_mlp"):
                if L[nm] is not None:
                    _want(L[nm], nm, torch.float32, 1)
            if (tuple(L["w_qkv"].shape) != (3 * width, width) or tuple(L["w_out"].shape) != (width, width)
                    or tuple(L["w_fc"].shape) != (inner, width) or tuple(L["w_mlp"].shape) != (width, inner)):
                raise KernelError("fused_decode_build: matrix shapes do not fit the sizes")
            keep += [L[k] for k in L if isinstance(L[k], torch.Tensor) and not k.startswith("w_")]
            packed = [packs.setdefault(L[nm].data_ptr(), pack_weight_units(L[nm]))
                      for nm in ("w_qkv", "w_out", "w_fc", "w_mlp")]      # a shared layer: once
            _check(lib.hs_decode_persistent_layer(
                c_void_p(base + i * lb), _ptr(packed[0]), _ptr(packed[1]), _ptr(packed[2]),
                _ptr(packed[3]), _ptr(L["b_qkv"]), _ptr(L["b_out"]), _ptr(L["b_fc"]),
                _ptr(L["b_mlp"]), _ptr(L["ln1_g"]), _ptr(L["ln1_b"]), _ptr(L["ln2_g"]),
                _ptr(L["ln2_b"]), float(L["eps1"]), float(L["eps2"]), float(L["scale"]),
                int(ACTIVATIONS[L["act"]]), int(width), int(inner),
                ctypes.c_longlong(int(L["entry"]) * rows_per_entry)), "decode_persistent_layer")
        _want(head_weight, "head_weight", torch.bfloat16, 2)
        head_packed = pack_weight_units(head_weight)
        keep += list(packs.values()) + [head_packed]
        _check(lib.hs_decode_persistent_tables(
            c_void_p(base + len(layers) * lb), _ptr(head_packed), int(vocab), int(width),
            _ptr(pool), ctypes.c_longlong(pool.shape[0] * rows_per_entry)),
            "decode_persistent_tables")
        dev = host.to(self.device)
        return FusedTables(dev, len(layers), lb, keep)

    def fused_decode(self, tables, *, wte, wpe, lnf_g, lnf_b, eps_f, width, inner, vocab,
                     n_heads, pool, num_pages, max_pages, x, qkv, att, u, logits, tokens,
                     feedback, tok_ids, tok_pos, tok_req, table, logit_rows, samp_slot,
                     plan_head, n_tokens, n_requests, n_logit_rows, status, stop_after=0):
        """One decode step of up to 16 single-query tokens in one persistent kernel: embedding,
        every layer, final norm, head, greedy tokens (``tokens[:n_logit_rows]``, the status
        word behind them).  Buffers are the caller's; scratch is this object's."""
        M, W = int(n_tokens), int(n_logit_rows)
        if not 0 < M <= self.FUSED_MAX_TOKENS or W > self.FUSED_MAX_TOKENS:
            raise KernelError(f"fused_decode: {M} tokens / {W} wanted rows exceed "
                              f"{self.FUSED_MAX_TOKENS}")
        _want(x, "x", torch.float32, 2)
        for t, nm, wd in ((qkv, "qkv", 3 * width), (att, "att", width), (u, "u", inner)):
            _want(t, nm, torch.bfloat16, 2)
            if t.shape[0] < M or t.shape[1] != wd:
                raise KernelError(f"fused_decode: {nm} has shape {tuple(t.shape)}")
        if x.shape[0] < M or x.shape[1] != width:
            raise KernelError("fused_decode: x does not fit")
        if W:
            _want(logits, "logits", torch.float32, 2)
            if logits.shape[0] < W or logits.shape[1] != vocab:
                raise KernelError("fused_decode: logits do not fit")
        _want(tokens, "tokens", torch.int32, 1)
        if tokens.shape[0] < W + 1:
            raise KernelError("fused_decode: tokens has no room for the status word")
        for t, nm in ((tok_ids, "tok_ids"), (tok_pos, "tok_pos"), (tok_req, "tok_req")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < M:
                raise KernelError(f"fused_decode: {nm} shorter than the tokens")
        _want(table, "table", torch.int32, 2)
        if table.shape[1] != max_pages:
            raise KernelError("fused_decode: block table width != max_pages")
        grid = self.lib.hs_decode_persistent_grid()
        if grid <= 0:
            raise KernelError("fused_decode: the kernel does not fit this device")
        S = self.lib.hs_decode_persistent_slices(int(n_requests), int(n_heads))
        acc = ml = None
        if S > 1:
            acc = self._scratch_buffer("fused_att_acc", M * n_heads * S * 64, torch.float32)
            ml = self._scratch_buffer("fused_att_ml", M * n_heads * S * 2, torch.float32)
        amax_v = self._scratch_buffer("fused_amax_val", grid * 16, torch.float32)
        amax_i = self._scratch_buffer("fused_amax_idx", grid * 16, torch.int32)
        sync = self._scratch_buffer("fused_sync", 4, torch.int32)
        self.launches += 1
        _check(self.lib.hs_decode_persistent(
            tables.layers_ptr, tables.tables_ptr, tables.n_layers, _ptr(wte), _ptr(wpe),
            _ptr(lnf_g), _ptr(lnf_b), float(eps_f), int(width), int(inner), int(vocab),
            int(n_heads), int(wpe.shape[0]), _ptr(pool), int(num_pages), int(max_pages), _ptr(x),
            _ptr(qkv), _ptr(att), _ptr(u), _ptr(logits), _ptr(acc), _ptr(ml), _ptr(amax_v),
            _ptr(amax_i), _ptr(tokens), _ptr(feedback), int(feedback.shape[0]), _ptr(tok_ids),
            _ptr(tok_pos), _ptr(tok_req), _ptr(table), _ptr(logit_rows), _ptr(samp_slot),
            _ptr(plan_head), M, W, W, S, _ptr(sync), _ptr(status), int(stop_after),
            self._stream()), "decode_persistent")

    # -- other norms, rotations, block-diagonal linears ---------------------------------
    def dyt_norm(self, out, x, weight, bias, alpha, rows=None):
        """out[i] = tanh(alpha * x[r]) * weight + bias with r = rows[i] if rows is given else i
        (a norm without statistics)."""
        _want(out, "out", _FLOATS, 2)
        _want(x, "x", torch.float32, 2)
        _want(weight, "weight", torch.float32, 1)
        _want(bias, "bias", torch.float32, 1)
        n, width = out.shape
        if x.shape[1] != width or weight.shape[0] != width or bias.shape[0] != width:
            raise KernelError("dyt_norm: widths of out, x, weight, bias differ")
        if rows is not None:
            _want(rows, "rows", torch.int32, 1)
            if rows.shape[0] < n:
                raise KernelError("dyt_norm: fewer row indices than output rows")
        elif x.shape[0] < n:
            raise KernelError("dyt_norm: x has fewer rows than out")
        self.launches += 1
        _check(self.lib.hs_dyt_norm(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(rows), n,
                                    width, float(alpha), _DT[out.dtype], self._stream()),
               f"dyt_norm(width={width})")

    def scale_(self, t, factor):
        """t *= factor, in place (float32)."""
        _want(t, "t", torch.float32)
        self.launches += 1
        _check(self.lib.hs_scale(_ptr(t), t.numel(), float(factor), self._stream()), "scale")

    def rotary_pairs(self, buf, tok_pos, tok_req, freq, *, n_vec, vec_stride, offset, dims):
        """Rotary positions on interleaved pairs, in place: in every row t of the float32
        ``buf``, the ``n_vec`` vectors at columns ``offset + v * vec_stride`` have the pairs
        (2i, 2i+1) of their first ``dims`` entries turned by ``tok_pos[t] * freq[i]``."""
        _want(buf, "buf", torch.float32, 2)
        _want(tok_pos, "tok_pos", torch.int32, 1)
        _want(tok_req, "tok_req", torch.int32, 1)
        _want(freq, "freq", torch.float32, 1)
        n, stride = buf.shape
        if dims % 2 or freq.shape[0] < dims // 2:
            raise KernelError("rotary_pairs: dims must be even and freq hold dims / 2 entries")
        if n_vec and offset + (n_vec - 1) * vec_stride + dims > stride:
            raise KernelError("rotary_pairs: the vectors exceed the row")
        if tok_pos.shape[0] < n or tok_req.shape[0] < n:
            raise KernelError("rotary_pairs: fewer positions than rows")
        self.launches += 1
        _check(self.lib.hs_rotary_pairs(_ptr(buf), _ptr(tok_pos), _ptr(tok_req), _ptr(freq), n,
                                        stride, n_vec, vec_stride, offset, dims, self._stream()),
               "rotary_pairs")

    def grouped_linear(self, out, a, w, *, a_offset=0, a_group_stride=None, w_nk=None,
                       exact=False):
        """Block-diagonal linear: ``out[t, g*n + j] = sum_k a[t, a_offset + g*a_group_stride + k]
        * w[g, k, j]``.  ``a`` float32 (a group's input may be a slice of a wider row), ``w``
        [groups, k, n] (k-major), ``out`` [T, groups * n] float32 or of w's type.  ``w_nk`` is
        the same weight as [groups, n, k] in bfloat16: with it, 64 tokens or more and k a
        multiple of 32, the product runs on the tensor cores (``a`` rounded to bfloat16; with
        ``exact`` ``a`` enters as the sum of three bfloat16 terms, which loses nothing of a
        float32: for weights that are bfloat16 numbers the result is then the float32 product,
        and ``out`` is float32)."""
        _want(a, "a", torch.float32, 2)
        _want(w, "w", _FLOATS, 3)
        _want(out, "out", _FLOATS, 2)
        groups, k, n = w.shape
        gs = k if a_group_stride is None else int(a_group_stride)
        T = out.shape[0]
        if out.shape[1] != groups * n or a.shape[0] < T:
            raise KernelError("grouped_linear: out does not fit the weights")
        if a_offset + (groups - 1) * gs + k > a.shape[1]:
            raise KernelError("grouped_linear: the groups' inputs exceed a's row")
        if out.dtype != torch.float32 and out.dtype != w.dtype:
            raise KernelError("grouped_linear: out is float32 or of the weights' type")
        self.launches += 1
        if (w_nk is not None and T >= 64 and w_nk.dtype == torch.bfloat16 and self.tensor_cores
                and tuple(w_nk.shape) == (groups, n, k) and w_nk.is_contiguous()):
            code = self.lib.hs_grouped_linear_mma(_ptr(out), _ptr(a), _ptr(w_nk), T, a.shape[1],
                                                  int(a_offset), gs, groups, n, k,
                                                  _DT[out.dtype], 3 if exact else 1,
                                                  self._stream())
            if code != -1:
                _check(code, f"grouped_linear_mma(groups={groups},n={n},k={k})")
                return
        _check(self.lib.hs_grouped_linear(_ptr(out), _ptr(a), _ptr(w), T, a.shape[1],
                                          int(a_offset), gs, groups, n, k, _DT[w.dtype],
                                          _DT[out.dtype], self._stream()),
               f"grouped_linear(groups={groups},n={n},k={k})")

    # -- attention over a shared latent ---------------------------------------------------
    def latent_append(self, pool, proj, norm_w, table, tok_pos, tok_req, *, c_offset, rank,
                      rot_dim, eps, page_size, status, freq=None, rot_dims=0):
        """Cache row of each token: ``[rms_norm(proj[t, c_offset : +rank]) * norm_w |
        proj[t, c_offset + rank : + rot_dim]]``; with ``freq`` the first ``rot_dims`` entries
        of the second part are rotated on the way (interleaved pairs, as ``rotary_pairs``),
        without it the part is taken as it stands.  ``pool`` is [pages, 1, 1, page_size,
        rank + rot_dim]."""
        _want(proj, "proj", torch.float32, 2)
        _want(pool, "pool", _FLOATS)
        _want(norm_w, "norm_w", torch.float32, 1)
        _want(table, "table", torch.int32, 2)
        n = proj.shape[0]
        W = rank + rot_dim
        if pool.numel() % (page_size * W) or norm_w.shape[0] != rank:
            raise KernelError("latent_append: pool or norm weight does not fit rank + rot_dim")
        if c_offset + W > proj.shape[1] or tok_pos.shape[0] < n or tok_req.shape[0] < n:
            raise KernelError("latent_append: rows do not fit")
        self.launches += 1
        _check(self.lib.hs_latent_append(_ptr(pool), _ptr(proj), _ptr(norm_w), _ptr(table),
                                         _ptr(tok_pos), _ptr(tok_req), n, proj.shape[1],
                                         int(c_offset), rank, rot_dim, float(eps), page_size,
                                         pool.numel() // (page_size * W), table.shape[1],
                                         _DT[pool.dtype], _ptr(status), _ptr(freq),
                                         int(rot_dims) if freq is not None else 0,
                                         self._stream()),
               "latent_append")

    def latent_attention(self, out, qa, qr, pool, table, tok_pos, tok_req, sink, *, n_heads,
                         rank, rot_dim, qr_head_stride, qr_offset, scale, page_size, status,
                         freq=None, rot_dims=0, plan=None):
        """Causal softmax attention with a sink over cache rows ``[c (rank) | kr (rot_dim)]``
        shared by all heads: score = (qa[t,h] . c + qr[t,h] . kr) * scale, the denominator
        also holds exp(sink[h]); ``out[t, h] = sum_j weight_j c_j`` ([T, n_heads * rank],
        float32).  ``qa`` [T, n_heads * rank] float32; head h's rotated query part is
        ``qr[t, qr_offset + h * qr_head_stride : + rot_dim]``; with ``freq`` it arrives
        unrotated and its first ``rot_dims`` entries are rotated as they are read.  With the
        step's ``plan`` and a bfloat16 cache, the plan's tiles (prompt portions) run on the
        tensor cores with the queries rounded to bfloat16, its single-query tokens on the CUDA
        cores; without a plan every token runs on the CUDA cores."""
        _want(out, "out", torch.float32, 2)
        _want(qa, "qa", torch.float32, 2)
        _want(qr, "qr", torch.float32, 2)
        _want(pool, "pool", _FLOATS)
        _want(table, "table", torch.int32, 2)
        _want(sink, "sink", torch.float32, 1)
        n = out.shape[0]
        W = rank + rot_dim
        if out.shape[1] != n_heads * rank or qa.shape[1] != n_heads * rank or qa.shape[0] < n:
            raise KernelError("latent_attention: out / qa are [T, n_heads * rank]")
        if qr.shape[0] < n or qr_offset + (n_heads - 1) * qr_head_stride + rot_dim > qr.shape[1]:
            raise KernelError("latent_attention: the rotated query parts exceed qr's row")
        if pool.numel() % (page_size * W) or sink.shape[0] != n_heads:
            raise KernelError("latent_attention: pool or sink does not fit")
        rot = int(rot_dims) if freq is not None else 0
        n_pages = pool.numel() // (page_size * W)
        listed = None
        if (plan is not None and plan.tile_cap > 0 and pool.dtype == torch.bfloat16
                and self.tensor_cores and self.latent_mma):
            code = self.lib.hs_latent_prefill_mma(
                _ptr(out), _ptr(qa), _ptr(qr), _ptr(pool), _ptr(table), _ptr(sink),
                _ptr(plan.data), 4 + plan_decode_ints(plan.n_rows), plan.tile_cap, n_heads, rank,
                rot_dim, qr.shape[1], int(qr_head_stride), int(qr_offset), float(scale),
                page_size, n_pages, table.shape[1], _ptr(status), _ptr(freq), rot,
                self._stream())
            if code != -1:
                _check(code, f"latent_prefill_mma(rank={rank},rot_dim={rot_dim})")
                self.launches += 1
                if plan.decode_cap == 0:
                    return
                listed = plan.data          # the CUDA-core kernel takes the single-query tokens
                n = plan.decode_cap
        # few tokens: the keys of each are split over several blocks so that the device fills
        blocks = n * -(-n_heads // 8)
        nsplit = 1 if blocks >= self.sm_count else min(16, -(-2 * self.sm_count // blocks))
        if self.latent_splits is not None:
            nsplit = int(self.latent_splits)
        partial = None
        if nsplit > 1:
            # shares are kept by flat token index, whichever tokens this launch works on
            partial = self._scratch_buffer("latent_partial",
                                           out.shape[0] * n_heads * nsplit * (rank + 2),
                                           torch.float32)
        self.launches += 2 if nsplit > 1 else 1
        _check(self.lib.hs_latent_attention(
            _ptr(out), _ptr(qa), _ptr(qr), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
            _ptr(sink), n, n_heads, rank, rot_dim, qr.shape[1], int(qr_head_stride),
            int(qr_offset), float(scale), page_size, n_pages,
            table.shape[1], _DT[pool.dtype], _ptr(status), nsplit, _ptr(partial), _ptr(freq),
            rot, _ptr(listed), self._stream()),
            f"latent_attention(rank={rank},rot_dim={rot_dim})")

    # -- the gated delta rule ---------------------------------------------------------------
    @staticmethod
    def _delta_sizes(shape):
        return (shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"], shape["taps"],
                shape["a_rank"], shape["g_rank"])

    def delta_prepare(self, qn, kn, vv, beta, decay, proj, conv_w, a2, dt_bias, a_log, state,
                      tok_req, req_start, req_len, req_slot, shape, z_a=None):
        """From the fused projection rows ``[q | k | v | b | a | g]`` (float32): short causal
        convolution and silu on q, k, v (history before a portion from ``state``), unit q and k
        per head (q also times dim^-1/2), beta = sigmoid(b), decay = exp(-exp(a_log) *
        softplus(a2 a + dt_bias)); then the convolution history in ``state`` moves on.
        ``z_a`` [T, heads * dim] float32, if given, is ``a2 a`` formed beforehand."""
        for t, nm in ((qn, "qn"), (kn, "kn"), (vv, "vv"), (beta, "beta"), (decay, "decay"),
                      (proj, "proj")):
            _want(t, nm, torch.float32, 2)
        for t, nm in ((conv_w, "conv_w"), (a2, "a2"), (dt_bias, "dt_bias"), (a_log, "a_log"),
                      (state, "state")):
            _want(t, nm, torch.float32)
        H, HK, D, V, taps, ra, rg = self._delta_sizes(shape)
        C = 2 * HK * D + H * V
        if proj.shape[1] != C + H + ra + rg:
            raise KernelError("delta_prepare: the projection row does not fit the sizes")
        if state[0].numel() != H * D * V + (taps - 1) * C:
            raise KernelError("delta_prepare: the state does not fit the sizes")
        self.launches += 2 if taps > 1 else 1
        _check(self.lib.hs_delta_prepare(
            _ptr(qn), _ptr(kn), _ptr(vv), _ptr(beta), _ptr(decay), _ptr(proj), _ptr(conv_w),
            _ptr(a2), _ptr(dt_bias), _ptr(a_log), _ptr(state), _ptr(tok_req), _ptr(req_start),
            _ptr(req_len), _ptr(req_slot), proj.shape[0], req_start.shape[0], H, HK, D, V, taps,
            ra, rg, _ptr(z_a), self._stream()), "delta_prepare")

    def delta_recurrence(self, o, state, qn, kn, vv, beta, decay, req_start, req_len, req_slot,
                         shape):
        """Per request and head, token after token on the float32 state S [dim, vdim]:
        S <- decay * S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
        H, HK, D, V, taps, ra, rg = self._delta_sizes(shape)
        for t, nm in ((o, "o"), (qn, "qn"), (kn, "kn"), (vv, "vv"), (beta, "beta"),
                      (decay, "decay")):
            _want(t, nm, torch.float32, 2)
        _want(state, "state", torch.float32)
        self.launches += 1
        _check(self.lib.hs_delta_recurrence(
            _ptr(o), _ptr(state), _ptr(qn), _ptr(kn), _ptr(vv), _ptr(beta), _ptr(decay),
            _ptr(req_start), _ptr(req_len), _ptr(req_slot), req_start.shape[0], H, HK, D, V,
            taps, ra, rg, self._stream()), f"delta_recurrence(dim={D},vdim={V})")

    def delta_finish(self, out, o, proj, g2, norm_w, tok_req, eps, shape, z_g=None):
        """out = o / sqrt(mean(o^2) + eps) per head * norm_w * sigmoid(g2^T g); ``g2`` is
        [g_rank, heads * vdim] (and ``a2`` of :meth:`delta_prepare` [a_rank, heads * dim])."""
        H, HK, D, V, taps, ra, rg = self._delta_sizes(shape)
        _want(out, "out", _FLOATS, 2)
        _want(o, "o", torch.float32, 2)
        _want(proj, "proj", torch.float32, 2)
        _want(g2, "g2", torch.float32, 2)
        _want(norm_w, "norm_w", torch.float32, 1)
        self.launches += 1
        _check(self.lib.hs_delta_finish(
            _ptr(out), _ptr(o), _ptr(proj), _ptr(g2), _ptr(norm_w), _ptr(tok_req), out.shape[0],
            float(eps), H, HK, D, V, taps, ra, rg, _DT[out.dtype], _ptr(z_g), self._stream()),
            "delta_finish")

    # -- routed feed-forward ---------------------------------------------------------------
    def moe_route(self, sel_idx, sel_w, h, w_router, tok_req, *, top, n_groups, keep, z=None):
        """Per token: sigmoid scores of float32 router logits, group-limited choice of ``top``
        experts, weights normalised over the chosen ones.  ``z`` [T, experts] float32, if given,
        holds the logits (formed as one matrix product over the step)."""
        _want(sel_idx, "sel_idx", torch.int32, 2)
        _want(sel_w, "sel_w", torch.float32, 2)
        _want(h, "h", _FLOATS, 2)
        _want(w_router, "w_router", torch.float32, 2)
        E, width = w_router.shape
        if h.shape[1] != width or sel_idx.shape[1] != top or sel_w.shape[1] != top:
            raise KernelError("moe_route: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_moe_route(_ptr(sel_idx), _ptr(sel_w), _ptr(h), _ptr(w_router),
                                     _ptr(tok_req), sel_idx.shape[0], width, E, top, n_groups,
                                     keep, _DT[h.dtype], _ptr(z), self._stream()),
               f"moe_route(experts={E},top={top},groups={n_groups},keep={keep})")

    def moe_experts(self, x, y, h, w_gate, w_up, w_down, sel_idx, sel_w, tok_req, *, limit,
                    act="clamped"):
        """x += sum over a token's chosen experts of weight * W_down act(W_gate h, W_up h) with
        act(g, u) = min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, +-limit) + 1)
        (``act="clamped"``) or silu(g) * u (``act="silu"``, no limit), or W_down relu(W_up h)^2
        for experts without a gate matrix (``act="relu2"``, ``w_gate`` None).
        Expert matrices stacked as stored: gate / up [E, ff, width], down [E, width, ff]; ``y``
        is float32 scratch [T * top, ff].  Many pairs in bfloat16 are sorted by expert on the
        device and run as tiles on the tensor cores; few pairs, and float32, as one
        matrix-vector product per pair."""
        _want(x, "x", torch.float32, 2)
        _want(y, "y", torch.float32, 2)
        _want(h, "h", _FLOATS, 2)
        if (w_gate is None) != (act == "relu2"):
            raise KernelError("moe_experts: experts have a gate matrix unless act is 'relu2'")
        for t, nm in ((w_gate, "w_gate"), (w_up, "w_up"), (w_down, "w_down")):
            if t is not None:
                _want(t, nm, h.dtype, 3)
        E, ff, width = w_up.shape
        T, top = sel_idx.shape
        if tuple(w_up.shape) != (E, ff, width) or tuple(w_down.shape) != (E, width, ff) \
                or h.shape[1] != width or x.shape[1] != width or y.shape[0] < T * top \
                or y.shape[1] != ff:
            raise KernelError("moe_experts: shapes do not fit")
        key = (T, width, ff, top, E, h.dtype)
        need = self._moe_need.get(key)
        if need is None:
            ni, nb = ctypes.c_longlong(0), ctypes.c_longlong(0)
            self.lib.hs_moe_sorted_scratch(T, width, ff, top, E, _DT[h.dtype], ctypes.byref(ni),
                                           ctypes.byref(nb))
            need = (ni.value, nb.value) if self.sorted_experts else (0, 0)
            self._moe_need[key] = need
        ints = rows = None
        if need[0]:
            ints = self._scratch_buffer("moe_ints", need[0], torch.int32)
            rows = self._scratch_buffer("moe_rows", need[1], torch.uint8)
        self.launches += 4 if ints is not None else 2
        _check(self.lib.hs_moe_experts(_ptr(x), _ptr(y), _ptr(h), _ptr(w_gate), _ptr(w_up),
                                       _ptr(w_down), _ptr(sel_idx), _ptr(sel_w), _ptr(tok_req),
                                       T, width, ff, top, E, float(limit),
                                       EXPERT_ACTIVATIONS[act], _DT[h.dtype],
                                       _ptr(ints), _ptr(rows), self._stream()),
               f"moe_experts(ff={ff})")

    def moe_route_top(self, sel_idx, sel_w, h, w_router, bias, tok_req, *, top, z=None):
        """Per token: float32 logits ``W_r h + bias``, the ``top`` largest (the lower index wins
        a tie), weights = softmax over the chosen logits alone.  ``z`` [T, experts] float32, if
        given, holds ``W_r h`` (formed as one matrix product over the step)."""
        _want(sel_idx, "sel_idx", torch.int32, 2)
        _want(sel_w, "sel_w", torch.float32, 2)
        _want(h, "h", _FLOATS, 2)
        _want(w_router, "w_router", torch.float32, 2)
        E, width = w_router.shape
        if bias is not None:
            _want(bias, "bias", torch.float32, 1)
            if bias.shape[0] != E:
                raise KernelError("moe_route_top: one bias per expert")
        if h.shape[1] != width or sel_idx.shape[1] != top or sel_w.shape[1] != top:
            raise KernelError("moe_route_top: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_moe_route_top(_ptr(sel_idx), _ptr(sel_w), _ptr(h), _ptr(w_router),
                                         _ptr(bias), _ptr(tok_req), sel_idx.shape[0], width, E,
                                         top, _DT[h.dtype], _ptr(z), self._stream()),
               f"moe_route_top(experts={E},top={top})")

    def gated_act(self, out, gu, h=None, w_s=None, tok_req=None, act="silu"):
        """out[t, f] = act(gu[t, f]) * gu[t, ff + f] (* sigmoid(h[t] . w_s), one number per
        token, when ``w_s`` is given): the middle of a gated feed-forward whose gate and up
        projections came as one product."""
        _want(out, "out", _FLOATS, 2)
        _want(gu, "gu", out.dtype, 2)
        T, ff = out.shape
        if gu.shape[1] != 2 * ff or gu.shape[0] < T:
            raise KernelError("gated_act: gu is [T, 2 * ff]")
        width = 0
        if w_s is not None:
            _want(h, "h", out.dtype, 2)
            _want(w_s, "w_s", out.dtype, 1)
            width = h.shape[1]
            if w_s.shape[0] != width or h.shape[0] < T:
                raise KernelError("gated_act: h and w_s do not fit")
        if act not in ACTIVATIONS:
            raise KernelError(f"gated_act: unknown activation {act!r}")
        self.launches += 1
        _check(self.lib.hs_gated_act(_ptr(out), _ptr(gu), _ptr(h), _ptr(w_s), _ptr(tok_req), T, ff,
                                     width, ACTIVATIONS[act], _DT[out.dtype], self._stream()),
               "gated_act")

    # -- root-mean-square norms ---------------------------------------------------------
    def rms_norm(self, out, x, weight, eps, rows=None, one_plus=False, gate=None, gate_offset=0):
        """out[i] = x[r] / sqrt(mean(x[r]^2) + eps) * weight (r = rows[i] or i; ``one_plus``:
        times 1 + weight); with ``gate`` (float32 [T, *]) also times
        sigmoid(gate[r, gate_offset + e]) per element."""
        _want(out, "out", _FLOATS, 2)
        _want(x, "x", torch.float32, 2)
        _want(weight, "weight", torch.float32, 1)
        n, width = out.shape
        if x.shape[1] != width or weight.shape[0] != width:
            raise KernelError("rms_norm: widths of out, x, weight differ")
        if rows is not None:
            _want(rows, "rows", torch.int32, 1)
            if rows.shape[0] < n:
                raise KernelError("rms_norm: fewer row indices than output rows")
        elif x.shape[0] < n:
            raise KernelError("rms_norm: x has fewer rows than out")
        g_stride = 0
        if gate is not None:
            _want(gate, "gate", torch.float32, 2)
            g_stride = gate.shape[1]
            if gate_offset + width > g_stride or gate.shape[0] < x.shape[0]:
                raise KernelError("rms_norm: the gate columns exceed the gate's row")
        self.launches += 1
        _check(self.lib.hs_rms_norm(_ptr(out), _ptr(x), _ptr(weight), _ptr(rows), n, width,
                                    float(eps), int(bool(one_plus)), _ptr(gate), int(gate_offset),
                                    g_stride, _DT[out.dtype], self._stream()),
               f"rms_norm(width={width})")

    def rms_norm_add(self, x, a, weight, eps, h=None, b=None, wa=None, wb=None, mix=0.5,
                     eps_in=None, ln=None):
        """The norm of a sublayer's output added into the stream: with y = a, or, given a second
        input, y = mix * (rms(a) * wa + rms(b) * wb) (those two norms with ``eps_in``, by
        default ``eps``):  x += rms(y) * weight, or x += y when ``weight`` is None.  ``h`` (of
        the compute type), if given, receives a copy of the new x, or with ``ln=(gamma, beta or
        None, eps)`` the layer norm of the new x."""
        _want(x, "x", torch.float32, 2)
        _want(a, "a", torch.float32, 2)
        n, width = x.shape
        if weight is not None:
            _want(weight, "weight", torch.float32, 1)
        if a.shape[0] < n or a.shape[1] != width or \
                (weight is not None and weight.shape[0] != width):
            raise KernelError("rms_norm_add: shapes do not fit")
        if b is not None:
            _want(b, "b", torch.float32, 2)
            _want(wa, "wa", torch.float32, 1)
            _want(wb, "wb", torch.float32, 1)
            if b.shape[0] < n or b.shape[1] != width or wa.shape[0] != width \
                    or wb.shape[0] != width:
                raise KernelError("rms_norm_add: the second input does not fit")
        if h is not None:
            _want(h, "h", _FLOATS, 2)
            if tuple(h.shape) != (n, width):
                raise KernelError("rms_norm_add: h has another shape than x")
        ln_g = None
        if ln is not None:
            if h is None:
                raise KernelError("rms_norm_add: the layer norm of the new rows goes to h")
            ln_g = _want(ln[0], "ln gamma", torch.float32, 1)
            if ln_g.shape[0] != width or (ln[1] is not None and ln[1].shape[0] != width):
                raise KernelError("rms_norm_add: the layer norm's parameters do not fit")
        self.launches += 1
        _check(self.lib.hs_rms_norm_add(_ptr(x), _ptr(h), _ptr(a), _ptr(wa), _ptr(b), _ptr(wb),
                                        float(mix), _ptr(weight), n, width,
                                        float(eps if eps_in is None else eps_in), float(eps),
                                        _DT[h.dtype] if h is not None else 0, _ptr(ln_g),
                                        _ptr(ln[1]) if ln is not None else None,
                                        float(ln[2]) if ln is not None else 0.0, self._stream()),
               f"rms_norm_add(width={width})")

    def cast_rows(self, out, x):
        """out = x (float32) rounded to bfloat16, elementwise."""
        _want(out, "out", torch.bfloat16)
        _want(x, "x", torch.float32)
        if out.numel() != x.numel():
            raise KernelError("cast_rows: sizes differ")
        self.launches += 1
        _check(self.lib.hs_cast_rows(_ptr(out), _ptr(x), x.numel(), self._stream()), "cast_rows")

    # -- attention with a distance bias, a score cap and a chunked mask --------------------
    def qk_prepare(self, q_out, pool, proj, wq, wk, table, tok_pos, tok_req, *, q_off, k_off,
                   v_off, eps, writes, n_heads, n_kv_heads, head_dim, page_size, status):
        """From float32 projection rows: queries RMS-normed over all ``n_heads * head_dim``
        entries at once (times ``wq``; None: as they are) into ``q_out``; keys normed likewise
        over ``n_kv_heads * head_dim`` (``wk``) into plane 0 of the token's page, values
        (columns at ``v_off``, or the un-normed keys when ``v_off`` is None) into plane 1.
        ``pool`` is [pages, 2, kv_heads, page_size, head_dim]."""
        _want(proj, "proj", torch.float32, 2)
        _want(q_out, "q_out", _FLOATS, 2)
        _want(pool, "pool", q_out.dtype)
        _want(table, "table", torch.int32, 2)
        n = q_out.shape[0]
        qw, kw = n_heads * head_dim, n_kv_heads * head_dim
        for t, nm, width in ((wq, "wq", qw), (wk, "wk", kw)):
            if t is not None:
                _want(t, nm, torch.float32, 1)
                if t.shape[0] != width:
                    raise KernelError(f"qk_prepare: {nm} has {t.shape[0]} entries, not {width}")
        if q_out.shape[1] != qw or proj.shape[0] < n or tok_pos.shape[0] < n or tok_req.shape[0] < n:
            raise KernelError("qk_prepare: rows do not fit")
        vo = -1 if v_off is None else int(v_off)
        if max(q_off + qw, k_off + kw, vo + kw if vo >= 0 else 0) > proj.shape[1]:
            raise KernelError("qk_prepare: the columns exceed the projection's row")
        per_page = 2 * n_kv_heads * page_size * head_dim
        if pool.numel() % per_page:
            raise KernelError("qk_prepare: the pool does not fit the sizes")
        self.launches += 1
        _check(self.lib.hs_qk_prepare(_ptr(q_out), _ptr(pool), _ptr(proj), _ptr(wq), _ptr(wk),
                                      _ptr(table), _ptr(tok_pos), _ptr(tok_req), n, proj.shape[1],
                                      int(q_off), int(k_off), vo, float(eps), int(bool(writes)),
                                      n_heads, n_kv_heads, head_dim, page_size,
                                      pool.numel() // per_page, table.shape[1], _DT[q_out.dtype],
                                      _ptr(status), self._stream()),
               f"qk_prepare(head_dim={head_dim})")

    def biased_attention(self, out, q, pool, table, tok_pos, tok_req, *, bias, gate, gate_offset,
                         n_heads, n_kv_heads, head_dim, page_size, scale, cap, chunk, window,
                         status, plan=None):
        """Causal softmax attention over the pages with score = cap * tanh(q . k * scale / cap)
        + bias[h, i - j] (``cap`` 0: none; ``bias`` float32 [heads, distances] or None), keys
        restricted to the query's chunk of ``chunk`` positions (0: none) and to the last
        ``window`` (0: all); head h's output is multiplied by sigmoid(gate[t, gate_offset + h])
        when ``gate`` (float32 [T, *]) is given.  With the step's ``plan`` and a bfloat16 cache
        the plan's tiles (prompt portions) run on the tensor cores and its single-query tokens
        on the CUDA cores; without a plan every token runs on the CUDA cores."""
        _want(out, "out", _FLOATS, 2)
        _want(q, "q", out.dtype, 2)
        _want(pool, "pool", out.dtype)
        _want(table, "table", torch.int32, 2)
        n = out.shape[0]
        if out.shape[1] != n_heads * head_dim or q.shape[1] != n_heads * head_dim or q.shape[0] < n:
            raise KernelError("biased_attention: out / q are [T, n_heads * head_dim]")
        n_dist = 0
        if bias is not None:
            _want(bias, "bias", torch.float32, 2)
            if bias.shape[0] != n_heads:
                raise KernelError("biased_attention: one row of biases per head")
            n_dist = bias.shape[1]
        g_stride = 0
        if gate is not None:
            _want(gate, "gate", torch.float32, 2)
            g_stride = gate.shape[1]
            if gate_offset + n_heads > g_stride or gate.shape[0] < n:
                raise KernelError("biased_attention: the gate columns exceed the gate's row")
        per_page = 2 * n_kv_heads * page_size * head_dim
        if pool.numel() % per_page:
            raise KernelError("biased_attention: the pool does not fit the sizes")
        num_pages = pool.numel() // per_page
        listed = head = None
        if (plan is not None and plan.tile_cap > 0 and out.dtype == torch.bfloat16
                and self.tensor_cores and self.biased_mma and plan.n_rows >= n):
            d = plan.data
            code = self.lib.hs_biased_attention_prefill(
                _ptr(out), _ptr(q), _ptr(pool), _ptr(table),
                _ptr(d[4 + plan_decode_ints(plan.n_rows):]), _ptr(d), plan.tile_cap,
                _ptr(self._scratch_buffer("biased_counter", 1, torch.int32)), _ptr(bias), n_dist,
                _ptr(gate), int(gate_offset), g_stride, n_heads, n_kv_heads, head_dim, page_size,
                num_pages, table.shape[1], float(scale), float(cap), int(chunk), int(window),
                _ptr(status), self._stream())
            if code != -1:
                _check(code, f"biased_attention_prefill(head_dim={head_dim})")
                self.launches += 1
                if plan.decode_cap == 0:
                    return
                listed, head = d[4:], d         # the CUDA-core kernel takes the single tokens
                n = plan.decode_cap
        self.launches += 1
        _check(self.lib.hs_biased_attention(
            _ptr(out), _ptr(q), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req), _ptr(bias),
            n_dist, _ptr(gate), int(gate_offset), g_stride, n, n_heads, n_kv_heads, head_dim,
            page_size, num_pages, table.shape[1], float(scale), float(cap),
            int(chunk), int(window), _DT[out.dtype], _ptr(listed), _ptr(head), _ptr(status),
            self._stream()),
            f"biased_attention(head_dim={head_dim})")

    # -- linear attention with a decay per head ---------------------------------------------
    def lightning_recurrence(self, o, state, proj, decay, req_start, req_len, req_slot, *, q_off,
                             k_off, v_off, heads, dim, vdim, act="silu", tok_pos=None, freq=None,
                             rot_dims=0, k_scale=1.0):
        """Per request and head, token after token on the float32 state S [dim, vdim] of the
        request's slot: S <- decay[h] S + k v^T; o = S^T q, with q, k, v = act(columns of the
        float32 projection rows ``proj``), laid out head by head from ``q_off``, ``k_off``,
        ``v_off``.  ``o`` is float32 [T, heads * vdim].  With ``freq`` (float32 [rot_dims / 2])
        q and k are turned by ``tok_pos`` on their first ``rot_dims`` numbers (number i pairs
        with i + rot_dims / 2) before they are used; k is multiplied by ``k_scale``."""
        _want(o, "o", torch.float32, 2)
        _want(proj, "proj", torch.float32, 2)
        _want(state, "state", torch.float32)
        _want(decay, "decay", torch.float32, 1)
        if decay.shape[0] != heads or o.shape[1] != heads * vdim:
            raise KernelError("lightning_recurrence: decay / o do not fit the heads")
        if state[0].numel() != heads * dim * vdim:
            raise KernelError("lightning_recurrence: the state does not fit the sizes")
        if max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim) > proj.shape[1]:
            raise KernelError("lightning_recurrence: the columns exceed the projection's row")
        if act not in ("none", "silu"):
            raise KernelError(f"lightning_recurrence: activation {act!r} not taken")
        if freq is None:
            rot_dims = 0
        elif rot_dims:
            _want(freq, "freq", torch.float32, 1)
            _want(tok_pos, "tok_pos", torch.int32, 1)
            if rot_dims % 2 or rot_dims > dim or freq.shape[0] < rot_dims // 2 \
                    or tok_pos.shape[0] < o.shape[0]:
                raise KernelError("lightning_recurrence: the rotated extent does not fit")
        # steps of many tokens: the activations in a pass of their own into compact rows, which
        # the recurrence then streams 16 bytes at a time (the same bits either way)
        T = o.shape[0]
        scratch = None
        if T >= self.lightning_bulk_rows and dim % 4 == 0 and vdim % 4 == 0:
            scratch = self._scratch_buffer("lightning_rows", T * (2 * heads * dim + heads * vdim),
                                           torch.float32)
        self.launches += 2 if scratch is not None else 1
        _check(self.lib.hs_lightning_recurrence(
            _ptr(o), _ptr(state), _ptr(proj), _ptr(decay), _ptr(req_start), _ptr(req_len),
            _ptr(req_slot), req_start.shape[0], T, proj.shape[1], int(q_off), int(k_off),
            int(v_off), heads, dim, vdim, ACTIVATIONS[act], _ptr(scratch),
            _ptr(tok_pos) if rot_dims else None, _ptr(freq) if rot_dims else None, int(rot_dims),
            float(k_scale), self._stream()),
            f"lightning_recurrence(dim={dim},vdim={vdim})")

    # -- norms behind a sublayer, a learned activation, capped logits -----------------------
    def layernorm_add(self, x, y, gamma, beta, eps, out=None, out_gamma=None, out_beta=None,
                      out_eps=None):
        """x += LayerNorm(y) * gamma + beta for the float32 rows of ``y`` (``beta`` may be
        None); with ``out``, also out = LayerNorm(new x) * out_gamma + out_beta: the rows the
        next sublayer takes, in the compute type (without ``out_gamma``: out = new x)."""
        _want(x, "x", torch.float32, 2)
        _want(y, "y", torch.float32, 2)
        _want(gamma, "gamma", torch.float32, 1)
        n, width = x.shape
        if y.shape[0] < n or y.shape[1] != width or gamma.shape[0] != width:
            raise KernelError("layernorm_add: shapes do not fit")
        for name, v in (("beta", beta), ("out_gamma", out_gamma), ("out_beta", out_beta)):
            if v is not None:
                _want(v, name, torch.float32, 1)
                if v.shape[0] != width:
                    raise KernelError(f"layernorm_add: {name} has another width")
        if out is not None:
            _want(out, "out", _FLOATS, 2)
            if tuple(out.shape) != (n, width):
                raise KernelError("layernorm_add: out needs x's shape")
        self.launches += 1
        _check(self.lib.hs_layernorm_add(
            _ptr(x), _ptr(y), _ptr(gamma), _ptr(beta), float(eps), _ptr(out), _ptr(out_gamma),
            _ptr(out_beta), float(eps if out_eps is None else out_eps), n, width,
            _DT[out.dtype] if out is not None else 0, self._stream()),
            f"layernorm_add(width={width})")

    def learned_act(self, out, z, act, values):
        """out = act(z) for an activation with learned numbers ``values``; z float32.
        xielu, values (p, q): z > 0: softplus(p) z^2 + z/2; else (1/2 + softplus(q))
        (e^z - 1 - z) + z/2."""
        a_pos, a_neg = learned_constants(act, values)
        _want(out, "out", _FLOATS)
        _want(z, "z", torch.float32)
        if out.numel() != z.numel():
            raise KernelError("learned_act: sizes differ")
        self.launches += 1
        _check(self.lib.hs_learned_act_xielu(_ptr(out), _ptr(z), z.numel(), a_pos, a_neg,
                                             _DT[out.dtype], self._stream()), "learned_act")

    def scale_softcap_(self, t, factor, cap):
        """t = cap * tanh(t * factor / cap), in place (float32)."""
        _want(t, "t", torch.float32)
        self.launches += 1
        _check(self.lib.hs_scale_softcap(_ptr(t), t.numel(), float(factor), float(cap),
                                         self._stream()), "scale_softcap")

    # -- the real-gated linear recurrent unit -----------------------------------------------
    def rglru_conv(self, u, proj, conv_w, conv_b, state, tok_req, req_start, req_slot, *, x_off,
                   channels, taps):
        """u[t, c] = conv_b[c] + sum_j conv_w[c, taps-1-j] * x[t-j, c], x = the columns
        ``x_off .. x_off + channels`` of the float32 rows ``proj``; rows before a request's
        first token of this step come from its slot of ``state`` ([slots, channels * taps]:
        the recurrence's state, then the last taps-1 inputs, oldest first)."""
        for name, v in (("u", u), ("proj", proj), ("conv_w", conv_w)):
            _want(v, name, torch.float32, 2)
        _want(conv_b, "conv_b", torch.float32, 1)
        _want(state, "state", torch.float32, 2)
        C, T = int(channels), u.shape[0]
        if u.shape[1] != C or tuple(conv_w.shape) != (C, taps) or conv_b.shape[0] != C \
                or x_off + C > proj.shape[1] or proj.shape[0] < T or state.shape[1] < C * taps:
            raise KernelError("rglru_conv: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_rglru_conv(_ptr(u), _ptr(proj), proj.shape[1], int(x_off),
                                      _ptr(conv_w), _ptr(conv_b), _ptr(state), state.shape[1],
                                      _ptr(tok_req), _ptr(req_start), _ptr(req_slot), T, C,
                                      int(taps), self._stream()), f"rglru_conv(channels={C})")

    def rglru_scan(self, out, state, u, z, proj, b_gates, rate, req_start, req_len, req_slot, *,
                   channels, blocks, taps, decay_scale, y_off, x_off):
        """Per request and channel, over the tokens of this step, on the float32 state of the
        request's slot: r, i = sigmoid(z + b_gates) (columns [part][r | i][channels/blocks]),
        log a = -decay_scale * r * rate, S <- a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(y);
        then the state and the convolution's last inputs are stored."""
        for name, v in (("u", u), ("z", z), ("proj", proj), ("state", state)):
            _want(v, name, torch.float32, 2)
        _want(out, "out", _FLOATS, 2)
        _want(b_gates, "b_gates", torch.float32, 1)
        _want(rate, "rate", torch.float32, 1)
        C = int(channels)
        if out.shape[1] != C or u.shape[1] != C or z.shape[1] != 2 * C or rate.shape[0] != C \
                or b_gates.shape[0] != 2 * C or state.shape[1] < C * taps \
                or max(y_off, x_off) + C > proj.shape[1]:
            raise KernelError("rglru_scan: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_rglru_scan(
            _ptr(out), _ptr(state), state.shape[1], _ptr(u), _ptr(z), _ptr(proj), proj.shape[1],
            int(y_off), int(x_off), _ptr(b_gates), _ptr(rate), _ptr(req_start), _ptr(req_len),
            _ptr(req_slot), req_start.shape[0], C, int(blocks), int(taps), float(decay_scale),
            _DT[out.dtype], self._stream()), f"rglru_scan(channels={C})")

    def rglru_step(self, out, state, proj, conv_w, conv_b, w_gates, b_gates, rate, tok_req,
                   req_slot, *, channels, blocks, taps, decay_scale, y_off, x_off) -> bool:
        """``rglru_conv``, the gates' block-diagonal product and ``rglru_scan`` for a step in
        which every request brings ONE token, in one launch and with the same bits.
        ``w_gates`` float32 [blocks, n, 2n].  False (nothing done) for parts of more than 256
        channels, which the three launches spread better over the device."""
        for name, v in (("proj", proj), ("state", state)):
            _want(v, name, torch.float32, 2)
        _want(out, "out", _FLOATS, 2)
        _want(w_gates, "w_gates", torch.float32, 3)
        C, n = int(channels), int(channels) // int(blocks)
        if out.shape[1] != C or tuple(w_gates.shape) != (blocks, n, 2 * n) or rate.shape[0] != C \
                or b_gates.shape[0] != 2 * C or state.shape[1] < C * taps \
                or max(y_off, x_off) + C > proj.shape[1] or conv_w.shape != (C, taps):
            raise KernelError("rglru_step: shapes do not fit")
        code = self.lib.hs_rglru_step(
            _ptr(out), _ptr(state), state.shape[1], _ptr(proj), proj.shape[1], int(y_off),
            int(x_off), _ptr(conv_w), _ptr(conv_b), _ptr(w_gates), _ptr(b_gates), _ptr(rate),
            _ptr(tok_req), _ptr(req_slot), out.shape[0], C, int(blocks), int(taps),
            float(decay_scale), _DT[out.dtype], self._stream())
        if code == -1:
            return False
        _check(code, f"rglru_step(channels={C})")
        self.launches += 1
        return True

    # -- attention over a window and pooled blocks --------------------------------------------
    def pooled_prepare(self, q_out, pool, proj, wq, wk, freq_qk, freq_v, table, tok_pos, tok_req,
                       *, n_heads, n_kv_heads, head_dim, value_dim, rot_dims, eps, writes,
                       page_size, status, coarse_pool=None, coarse_table=None, block=0):
        """From the float32 rows [q | k | v] of ``proj``: per-head RMS norms of q and k
        (weights ``wq``, ``wk`` or None), rotation of their first ``rot_dims`` numbers by the
        position (pairs d, d + rot_dims/2), rotation of the values over all of value_dim
        (``freq_v`` or None); q to ``q_out`` (float32), and with ``writes`` the row [k | v] of
        every key/value head into the token's page."""
        _want(q_out, "q_out", torch.float32, 2)
        _want(proj, "proj", torch.float32, 2)
        _want(pool, "pool", _FLOATS)
        _want(table, "table", torch.int32, 2)
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        if q_out.shape[1] != H * D or proj.shape[1] < (H + G) * D + G * V:
            raise KernelError("pooled_prepare: the rows do not fit the heads")
        num_pages = pool.numel() // (G * page_size * (D + V))
        cmax = cnum = 0
        if coarse_pool is not None:
            # only for steps in which every request brings ONE token: a token that completes a
            # block then forms the block's mean row here (``pooled_means`` is not needed)
            _want(coarse_pool, "coarse_pool", pool.dtype)
            _want(coarse_table, "coarse_table", torch.int32, 2)
            cmax, cnum = coarse_table.shape[1], coarse_pool.numel() // (G * page_size * (D + V))
        self.launches += 1
        _check(self.lib.hs_pooled_prepare(
            _ptr(q_out), _ptr(pool), _ptr(proj), proj.shape[1], _ptr(wq), _ptr(wk),
            _ptr(freq_qk), _ptr(freq_v), _ptr(table), table.shape[1], num_pages, _ptr(tok_pos),
            _ptr(tok_req), q_out.shape[0], H, G, D, V, int(rot_dims), float(eps), int(page_size),
            int(bool(writes)), _DT[pool.dtype], _ptr(coarse_pool), _ptr(coarse_table), cmax, cnum,
            int(block), _ptr(status), self._stream()),
            f"pooled_prepare(head_dim={D},value_dim={V})")

    def pooled_means(self, coarse_pool, coarse_table, pool, table, tok_pos, tok_req, *,
                     n_kv_heads, row, block, page_size, status):
        """For every token whose position completes a block of ``block`` positions: the mean of
        the block's rows as ``pool`` holds them, written as row ``position // block`` of the
        companion pool."""
        _want(coarse_pool, "coarse_pool", pool.dtype)
        _want(pool, "pool", _FLOATS)
        _want(table, "table", torch.int32, 2)
        _want(coarse_table, "coarse_table", torch.int32, 2)
        per_page = n_kv_heads * page_size * row
        self.launches += 1
        _check(self.lib.hs_pooled_means(
            _ptr(coarse_pool), _ptr(coarse_table), coarse_table.shape[1],
            coarse_pool.numel() // per_page, _ptr(pool), _ptr(table), table.shape[1],
            pool.numel() // per_page, _ptr(tok_pos), _ptr(tok_req), tok_pos.shape[0],
            int(n_kv_heads), int(row), int(block), int(page_size), _DT[pool.dtype], _ptr(status),
            self._stream()), f"pooled_means(block={block})")

    def pooled_attention(self, out, q, pool, table, coarse_pool, coarse_table, tok_pos, tok_req,
                         freq_v, *, n_heads, n_kv_heads, head_dim, value_dim, window, block,
                         scale, page_size, status, plan=None):
        """Per token at position i and query head: one softmax over the mean rows of the blocks
        b with b * block + block - 1 <= i - window and the token rows j with 0 <= i - j <
        window; the output turned back by -i over value_dim (``freq_v`` or None).  With the
        step's ``plan`` and a bfloat16 cache the plan's tiles (prompt portions) run on the
        tensor cores and its single-query tokens on the CUDA cores; without a plan, in float32
        and for sizes the tile kernel does not take every token runs on the CUDA cores."""
        _want(out, "out", _FLOATS, 2)
        _want(q, "q", torch.float32, 2)
        _want(pool, "pool", _FLOATS)
        _want(coarse_pool, "coarse_pool", pool.dtype)
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        T = out.shape[0]
        if out.shape[1] != H * V or q.shape[1] != H * D or q.shape[0] < T:
            raise KernelError("pooled_attention: the rows do not fit the heads")
        if out.dtype != pool.dtype:
            raise KernelError("pooled_attention: out has the cache's type")
        per_page = G * page_size * (D + V)
        listed = head = None
        if (plan is not None and plan.tile_cap > 0 and out.dtype == torch.bfloat16
                and self.tensor_cores and self.pooled_mma and plan.n_rows >= T):
            d = plan.data
            code = self.lib.hs_pooled_attention_prefill(
                _ptr(out), _ptr(q), _ptr(pool), _ptr(table), table.shape[1],
                pool.numel() // per_page, _ptr(coarse_pool), _ptr(coarse_table),
                coarse_table.shape[1], coarse_pool.numel() // per_page,
                _ptr(d[4 + plan_decode_ints(plan.n_rows):]), _ptr(d), plan.tile_cap,
                _ptr(self._scratch_buffer("pooled_counter", 1, torch.int32)), _ptr(freq_v), H, G,
                D, V, int(window), int(block), float(scale), int(page_size), _ptr(status),
                self._stream())
            if code != -1:
                _check(code, f"pooled_attention_prefill(head_dim={D},value_dim={V})")
                self.launches += 1
                if plan.decode_cap == 0:
                    return
                listed, head = d[4:], d         # the CUDA-core kernel takes the single tokens
                T = plan.decode_cap
        self.launches += 1
        _check(self.lib.hs_pooled_attention(
            _ptr(out), _ptr(q), _ptr(pool), _ptr(table), table.shape[1], pool.numel() // per_page,
            _ptr(coarse_pool), _ptr(coarse_table), coarse_table.shape[1],
            coarse_pool.numel() // per_page, _ptr(tok_pos), _ptr(tok_req), _ptr(freq_v), T, H, G,
            D, V, int(window), int(block), float(scale), int(page_size), _DT[pool.dtype],
            _DT[out.dtype], _ptr(listed), _ptr(head), _ptr(status), self._stream()),
            f"pooled_attention(head_dim={D},value_dim={V})")

    # -- time mixing, head norms, token-indexed tables ---------------------------------------
    def token_shift_mix(self, out, x, mu, state, tok_req, req_start, req_len, req_slot, *,
                        state_offset):
        """out[s, t] = x[t] + (x'[t] - x[t]) * mu[s] for every stream s (``mu`` float32
        [streams, width]), x' being the row before in the request; for a request's first row of
        the step it is the float32 row kept at ``state[slot, state_offset:]``, which then
        receives the step's last row of the request."""
        _want(out, "out", _FLOATS, 3)
        _want(x, "x", out.dtype, 2)
        _want(mu, "mu", torch.float32, 2)
        _want(state, "state", torch.float32, 2)
        S, T, W = out.shape
        if x.shape[0] < T or x.shape[1] != W or tuple(mu.shape) != (S, W) \
                or state_offset + W > state.shape[1]:
            raise KernelError("token_shift_mix: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_token_shift_mix(
            _ptr(out), _ptr(x), _ptr(mu), _ptr(state), state.shape[1], int(state_offset),
            _ptr(tok_req), _ptr(req_start), _ptr(req_len), _ptr(req_slot), T, W, S,
            _DT[out.dtype], self._stream()), "token_shift_mix")

    def timemix_decay(self, out, low, w2t, w0):
        """out[t, c] = exp(-exp(sum_j w2t[j, c] tanh(low[t, j]) + w0[c])), all float32; ``w2t``
        is the second matrix of the decay transposed, [inner, channels]."""
        _want(out, "out", torch.float32, 2)
        _want(low, "low", torch.float32, 2)
        _want(w2t, "w2t", torch.float32, 2)
        _want(w0, "w0", torch.float32, 1)
        T, C = out.shape
        rank = low.shape[1]
        if low.shape[0] < T or tuple(w2t.shape) != (rank, C) or w0.shape[0] != C:
            raise KernelError("timemix_decay: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_timemix_decay(_ptr(out), _ptr(low), _ptr(w2t), _ptr(w0), T, C, rank,
                                         self._stream()), f"timemix_decay(rank={rank})")

    def timemix_recurrence(self, o, state, r, k, v, w, u, req_start, req_len, req_slot, *, heads,
                           dim):
        """Per request and head, token after token on the float32 state S [dim, dim] at the
        start of the request's slot: o = (S + diag(u) k v^T)^T r, then S <- diag(w) S + k v^T.
        r, k, v, w, o: float32 [T, heads * dim]; u: float32 [heads * dim]."""
        T = o.shape[0]
        for t, nm in ((o, "o"), (r, "r"), (k, "k"), (v, "v"), (w, "w")):
            _want(t, nm, torch.float32, 2)
            if t.shape[0] < T or t.shape[1] != heads * dim:
                raise KernelError(f"timemix_recurrence: {nm} is [T, heads * dim]")
        _want(u, "u", torch.float32, 1)
        _want(state, "state", torch.float32, 2)
        if u.shape[0] != heads * dim or state.shape[1] < heads * dim * dim:
            raise KernelError("timemix_recurrence: u / state do not fit the sizes")
        self.launches += 1
        _check(self.lib.hs_timemix_recurrence(
            _ptr(o), _ptr(state), state.shape[1], _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u),
            _ptr(req_start), _ptr(req_len), _ptr(req_slot), req_start.shape[0], T, heads, dim,
            self._stream()), f"timemix_recurrence(dim={dim})")

    def head_norm_gate(self, out, o, weight, gate, *, gate_offset, heads, dim, eps,
                       gate_act="silu", out_scale=1.0):
        """out[t, h] = o[t, h] / rms(o[t, h]) (* weight) * act(gate columns) * out_scale for
        every head h of ``dim`` numbers; ``gate`` is float32 [T, *] with the head's columns from
        ``gate_offset`` on, ``gate_act`` silu or sigmoid; weight and gate may be None."""
        _want(out, "out", _FLOATS, 2)
        _want(o, "o", torch.float32, 2)
        T = out.shape[0]
        if out.shape[1] != heads * dim or o.shape[1] != heads * dim or o.shape[0] < T:
            raise KernelError("head_norm_gate: out / o are [T, heads * dim]")
        if weight is not None:
            _want(weight, "weight", torch.float32, 1)
            if weight.shape[0] != heads * dim:
                raise KernelError("head_norm_gate: one weight per number")
        g_stride = 0
        if gate is not None:
            _want(gate, "gate", torch.float32, 2)
            g_stride = gate.shape[1]
            if gate.shape[0] < T or gate_offset + heads * dim > g_stride:
                raise KernelError("head_norm_gate: the gate columns exceed the gate's row")
        if gate_act not in ("silu", "sigmoid"):
            raise KernelError(f"head_norm_gate: gate activation {gate_act!r} not taken")
        self.launches += 1
        _check(self.lib.hs_head_norm_gate(
            _ptr(out), _ptr(o), _ptr(weight), _ptr(gate), g_stride, int(gate_offset), T, heads,
            dim, float(eps), int(gate_act == "silu"), float(out_scale), _DT[out.dtype],
            self._stream()), f"head_norm_gate(dim={dim})")

    def gather_mul(self, out, g, table, tok_ids, tok_req, *, col_offset, feedback=None):
        """out[t, c] = g[t, c] * table[token[t], col_offset + c] (``g`` float32, ``out`` and
        ``table`` in the compute type); a token id -(s + 1) stands for ``feedback[s]``."""
        _want(out, "out", _FLOATS, 2)
        _want(g, "g", torch.float32, 2)
        _want(table, "table", out.dtype, 2)
        T, dim = out.shape
        if g.shape[0] < T or g.shape[1] != dim or col_offset + dim > table.shape[1]:
            raise KernelError("gather_mul: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_gather_mul(
            _ptr(out), _ptr(g), _ptr(table), table.shape[0], table.shape[1], _ptr(tok_ids),
            _ptr(tok_req), _ptr(feedback), 0 if feedback is None else feedback.shape[0], T, dim,
            int(col_offset), _DT[out.dtype], _DT[table.dtype], _ptr(self._status_of(tok_ids)),
            self._stream()), "gather_mul")

    def moe_route_table(self, sel_idx, sel_w, table, tok_ids, tok_req, *, top, feedback=None,
                        experts=None):
        """sel_idx[t] = table[token[t], :top] (int32 [rows, top]), sel_w = 1 / top."""
        _want(sel_idx, "sel_idx", torch.int32, 2)
        _want(sel_w, "sel_w", torch.float32, 2)
        _want(table, "table", torch.int32, 2)
        if table.shape[1] != top or sel_idx.shape[1] != top or sel_w.shape[1] != top:
            raise KernelError("moe_route_table: shapes do not fit")
        self.launches += 1
        _check(self.lib.hs_moe_route_table(
            _ptr(sel_idx), _ptr(sel_w), _ptr(table), table.shape[0], _ptr(tok_ids), _ptr(tok_req),
            _ptr(feedback), 0 if feedback is None else feedback.shape[0], sel_idx.shape[0], top,
            int(experts) if experts else 0x7fffffff, _ptr(self._status_of(tok_ids)),
            self._stream()), f"moe_route_table(top={top})")

    def _status_of(self, like):
        """A status word for kernels whose part hands none in: the engine's own when the runner
        has set it (``self.status``), else a private one."""
        st = getattr(self, "status", None)
        if st is None:
            st = self._scratch_buffer("own_status", 1, torch.int32)
        return st

    # -- attention with a distance slope, a window and kept first tokens ---------------------
    def span_prepare(self, q_out, pool, proj, table, tok_pos, tok_req, *, n_heads, n_kv_heads,
                     head_dim, value_dim, q_off, k_off, v_off, qk_norm, eps, writes, page_size,
                     status):
        """From float32 projection rows: q (columns from ``q_off``) to ``q_out`` (float32), and
        with ``writes`` the row [k | v] of every key/value head into the token's page; with
        ``qk_norm`` q and k are divided by their root mean square per head first.  ``v_off``
        None: the values are the keys as projected (before the norm).  ``pool`` is
        [pages, kv_heads, page_size, head_dim + value_dim]."""
        _want(q_out, "q_out", torch.float32, 2)
        _want(proj, "proj", torch.float32, 2)
        _want(pool, "pool", _FLOATS)
        _want(table, "table", torch.int32, 2)
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        if q_out.shape[1] != H * D or proj.shape[0] < q_out.shape[0]:
            raise KernelError("span_prepare: the rows do not fit the heads")
        if writes and k_off is None:
            raise KernelError("span_prepare: a layer that writes its rows has key columns")
        self.launches += 1
        _check(self.lib.hs_span_prepare(
            _ptr(q_out), _ptr(pool), _ptr(proj), proj.shape[1], int(q_off),
            -1 if k_off is None else int(k_off), -1 if v_off is None else int(v_off), _ptr(table),
            table.shape[1], pool.numel() // (G * page_size * (D + V)), _ptr(tok_pos),
            _ptr(tok_req), q_out.shape[0], H, G, D, V, int(bool(qk_norm)), float(eps),
            int(page_size), int(bool(writes)), _DT[pool.dtype], _ptr(status), self._stream()),
            f"span_prepare(head_dim={D},value_dim={V})")

    def span_attention(self, out, q, pool, table, tok_pos, tok_req, *, n_heads, n_kv_heads,
                       head_dim, value_dim, scale, slopes, window, keep_first, gate, gate_offset,
                       out_scale, page_size, status, plan=None):
        """Per token at position i and query head h: softmax over the keys j <= i with
        i - j < window (0: all) or j < keep_first of (q . k) * scale - slopes[h] * (i - j)
        (``slopes`` float32 [heads] or None); the head's output times sigmoid(gate[t,
        gate_offset + h * value_dim + e]) (``gate`` float32 [T, *] or None) times
        ``out_scale``.  With the step's ``plan`` and a bfloat16 cache the plan's tiles (prompt
        portions) run on the tensor cores and its single-query tokens on the CUDA cores;
        without a plan, in float32 and for sizes the tile kernel does not take every token
        runs on the CUDA cores."""
        _want(out, "out", _FLOATS, 2)
        _want(q, "q", torch.float32, 2)
        _want(pool, "pool", out.dtype)
        _want(table, "table", torch.int32, 2)
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        T = out.shape[0]
        if out.shape[1] != H * V or q.shape[1] != H * D or q.shape[0] < T:
            raise KernelError("span_attention: the rows do not fit the heads")
        if slopes is not None:
            _want(slopes, "slopes", torch.float32, 1)
            if slopes.shape[0] != H:
                raise KernelError("span_attention: one slope per head")
        g_stride = 0
        if gate is not None:
            _want(gate, "gate", torch.float32, 2)
            g_stride = gate.shape[1]
            if gate.shape[0] < T or gate_offset + H * V > g_stride:
                raise KernelError("span_attention: the gate columns exceed the gate's row")
        per_page = G * page_size * (D + V)
        num_pages = pool.numel() // per_page
        listed = head = None
        if (plan is not None and plan.tile_cap > 0 and out.dtype == torch.bfloat16
                and self.tensor_cores and self.span_mma and plan.n_rows >= T):
            d = plan.data
            code = self.lib.hs_span_attention_prefill(
                _ptr(out), _ptr(q), _ptr(pool), _ptr(table), table.shape[1], num_pages,
                _ptr(d[4 + plan_decode_ints(plan.n_rows):]), _ptr(d), plan.tile_cap,
                _ptr(self._scratch_buffer("span_counter", 1, torch.int32)), _ptr(slopes),
                _ptr(gate), g_stride, int(gate_offset), float(out_scale), H, G, D, V, int(window),
                int(keep_first), float(scale), int(page_size), _ptr(status), self._stream())
            if code != -1:
                _check(code, f"span_attention_prefill(head_dim={D},value_dim={V})")
                self.launches += 1
                if plan.decode_cap == 0:
                    return
                listed, head = d[4:], d         # the CUDA-core kernel takes the single tokens
                T = plan.decode_cap
        self.launches += 1
        _check(self.lib.hs_span_attention(
            _ptr(out), _ptr(q), _ptr(pool), _ptr(table), table.shape[1], num_pages, _ptr(tok_pos),
            _ptr(tok_req), _ptr(slopes), _ptr(gate), g_stride, int(gate_offset), float(out_scale),
            T, H, G, D, V, int(window), int(keep_first), float(scale), int(page_size),
            _DT[pool.dtype], _DT[out.dtype], _ptr(listed), _ptr(head), _ptr(status),
            self._stream()), f"span_attention(head_dim={D},value_dim={V})")

    # -- sampling ---------------------------------------------------------------
    def argmax(self, out, logits):
        _want(out, "out", torch.int32, 1)
        _want(logits, "logits", torch.float32, 2)
        rows, vocab = logits.shape
        if out.shape[0] < rows:
            raise KernelError("argmax: out shorter than the rows")
        self.launches += 1
        _check(self.lib.hs_argmax(_ptr(out), _ptr(logits), rows, vocab, self._stream()), "argmax")

    def sample(self, out, logits, temperature, top_k, seed_lo, seed_hi, position,
               feedback=None, feedback_slot=None, status_word=None):
        """Per row: argmax if temperature <= 0, else a draw from softmax(logits/temperature)
        restricted to the top_k largest when 0 < top_k < vocab.  With ``feedback`` and
        ``feedback_slot`` row i also stores its token to ``feedback[feedback_slot[i]]`` (slots
        below zero are skipped).  With ``status_word`` (one int32 on the device) its value is
        stored to ``out[rows]``: the engine's status travels behind the tokens."""
        _want(out, "out", torch.int32, 1)
        _want(logits, "logits", torch.float32, 2)
        rows, vocab = logits.shape
        _want(temperature, "temperature", torch.float32, 1)
        for t, nm in ((top_k, "top_k"), (seed_lo, "seed_lo"), (seed_hi, "seed_hi"),
                      (position, "position")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < rows:
                raise KernelError(f"sample: {nm} shorter than the rows")
        if out.shape[0] < rows or temperature.shape[0] < rows:
            raise KernelError("sample: out/temperature shorter than the rows")
        if (feedback is None) != (feedback_slot is None):
            raise KernelError("sample: feedback and feedback_slot come together")
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
            _want(feedback_slot, "feedback_slot", torch.int32, 1)
            if feedback_slot.shape[0] < rows:
                raise KernelError("sample: feedback_slot shorter than the rows")
        if status_word is not None:
            _want(status_word, "status_word", torch.int32, 1)
            if out.shape[0] < rows + 1:
                raise KernelError("sample: out has no room for the status word")
        self.launches += 1
        _check(self.lib.hs_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(top_k),
                                  _ptr(seed_lo), _ptr(seed_hi), _ptr(position), rows, vocab,
                                  _ptr(feedback), _ptr(feedback_slot), _ptr(status_word),
                                  self._stream()), "sample")
