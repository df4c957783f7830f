"""The device-side environment parts run in: device, precision mode, matrix products, scratch.

Two modes exist. "bfloat16" is what serving uses: bfloat16 weights, activations and cache,
float32 residual stream, norms, softmax and accumulation, tcgen05 tensor-core products.
"float32" is the true 32-bit path: every tensor and every product in IEEE float32 (FMA, no
tensor-core mode of reduced precision). The reference has no such path; its closest is
`gemm_fp32` with bfloat16 weights (crates/specrt/graphs/decoder.toml:174-278).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.runtime_options import RuntimeOptions
from ..kernels import lib as L
from ..kernels import ops

MODES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


class DeviceStatusError(RuntimeError):
    """A kernel reported a fault through the status word (bad page, bad token, a wait that ran out)."""


@dataclass
class LinearWeights:
    """A [N, K] matrix prepared for the runtime's mode, plus whatever its kernel caches for it."""
    weight: torch.Tensor
    n: int
    k: int
    plan: Optional[object] = None  # kernel-side descriptor cache


class Runtime:
    def __init__(self, device="cuda:0", dtype: Optional[str] = None, gemm: Optional[str] = None, options: Optional[RuntimeOptions] = None):
        """`options` holds every choice of kernel and fusion; `dtype` and `gemm` given here replace its fields."""
        if dtype is not None and dtype not in MODES:
            raise ValueError(f"dtype must be one of {sorted(set(MODES))}, got {dtype!r}")
        self.options = (options or RuntimeOptions()).merged(dtype=dtype, gemm=gemm)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise L.KernelLibraryError("the engine runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise L.KernelLibraryError("no CUDA device is visible; the engine has no CPU path")
        self.lib = L.load()
        self.device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.mode = self.options.dtype
        self.act_dtype = MODES[self.mode]
        self.gemm = self.options.gemm  # "auto" | "simt" | "tcgen05"
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.activate()

    def activate(self) -> None:
        """Make this runtime the one whose settings the kernel library uses: the device whose current stream kernels
        are launched on, programmatic dependent launch on or off, and the limit of bounded waits. The library keeps
        these per process, so every step (and every graph capture) calls this first; it costs three C calls."""
        ops._device_index = self.device_index
        self.lib.ib_set_pdl(1 if self.options.pdl else 0)
        self.lib.ib_set_wait_limit_ms(int(self.options.wait_limit_ms))

    # ---------------------------------------------------------------- memory
    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.act_dtype, device=self.device)

    def upload(self, t: torch.Tensor, dtype=None) -> torch.Tensor:
        t = t.to(self.device, non_blocking=False)
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        return t.contiguous()

    # ---------------------------------------------------------------- weights
    def matrix(self, w: torch.Tensor) -> LinearWeights:
        """Prepare a [N, K] matrix: float32 mode keeps every bit (bfloat16 widens exactly);
        bfloat16 mode rounds a 32-bit matrix to bfloat16, as the reference does at load
        (crates/specrt/src/weights.rs:388-396)."""
        w = self.upload(w, self.act_dtype)
        return LinearWeights(w, w.shape[0], w.shape[1])

    def vector(self, w: torch.Tensor) -> torch.Tensor:
        """Norm scales are used in float32 in both modes."""
        return self.upload(w, torch.float32)

    # ---------------------------------------------------------------- matrix product
    def linear(self, x: torch.Tensor, lw: LinearWeights, allow_split: bool = True, add_to: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """x [T, K] in the activation dtype -> partial products float32 [P, T, N]; their sum over P,
        taken in order, is x @ W^T. With `add_to` (float32 [T, N], the residual stream) a kernel that
        can add the product in its epilogue does so in place and None is returned: nothing is left
        to add. Otherwise the partial products come back as usual and `add_to` is untouched."""
        T = x.shape[0]
        if x.shape[1] != lw.k:
            raise L.KernelError(f"linear: x has {x.shape[1]} columns, the matrix has {lw.k}")
        use_tc = self.mode == "bfloat16" and self.gemm != "simt"
        if use_tc:
            from ..kernels import gemm_tcgen05
            if gemm_tcgen05.supports(lw.k):
                return gemm_tcgen05.linear(self, x, lw, allow_split, add_to)
            if self.gemm == "tcgen05":
                raise L.KernelError(f"linear: K={lw.k} is not a multiple of 8, which the tcgen05 kernel needs")
        out = self.empty((1, T, lw.n), torch.float32)
        ops.gemm_simt(x, lw.weight, out[0])
        return out

    def gate_up_act(self, x: torch.Tensor, lw: LinearWeights) -> torch.Tensor:
        """x [T, K] -> silu(x gate^T) * (x up^T) in the activation dtype, [T, I], for a matrix
        [2I, K] of gate rows then up rows. Enough bfloat16 tokens run as one tensor-core kernel
        whose epilogue applies the activation; otherwise the product and the SiLU-mul kernel."""
        T, inter = x.shape[0], lw.n // 2
        if self.mode == "bfloat16" and self.gemm != "simt":
            from ..kernels import gemm_tcgen05
            if self.options.swiglu_epilogue and gemm_tcgen05.swiglu_supported(T, lw.k, inter):
                act = self.empty((T, inter))
                gemm_tcgen05.gemm_swiglu(x, lw.weight, act, self.status, pair_min_tokens=self.options.pair_min_tokens)
                return act
        gu = self.linear(x, lw)
        act = self.empty((T, inter))
        ops.silu_mul(gu, act)
        return act

    # ---------------------------------------------------------------- status word
    def check_status(self) -> None:
        """Read the status word (synchronises) and raise if a kernel reported a fault."""
        self.raise_for(int(self.status.item()))

    def raise_for(self, bits: int) -> None:
        """Raise DeviceStatusError for a non-zero value of the status word (already on the host, for instance from the
        transfer that brought a step's tokens) and clear the word on the device."""
        if bits:
            self.status.zero_()
            what = [name for bit, name in ((L.ERR_BAD_PAGE, "a block table entry was missing or out of range"),
                                           (L.ERR_BAD_TOKEN, "a token id was outside the vocabulary"),
                                           (L.ERR_WAIT_TIMEOUT, "a bounded wait inside a kernel ran out"),
                                           (L.ERR_INTERNAL, "a kernel found one of its own assumptions broken")) if bits & bit]
            raise DeviceStatusError("; ".join(what) or f"status bits {bits}")
