"""Decode-ahead for the large-batch band: the next layer's weight is decoded on a side stream while
the current layer's GEMM runs.

In the large-batch band an ``NPVQLinear`` decodes its weight into a temporary dense matrix and
runs the dense tensor-core GEMM (the reference's ``_forward_dequant_gemm``,
neuropress/nn/np_vq_linear.py:1127-1148, does the two steps back to back on one stream).  The
decode does not depend on the activations, only on the weight, so it can run early: under the
GEMM of the layer before.  The two kernels want different parts of the SM (the decode is bound by
codebook gathers through L1, the GEMM by the tensor pipe and the power limit); where the GEMM's
ring leaves a few KiB of shared memory unclaimed (tile width 224 on CTA pairs) the decode's CTAs
are resident beside the GEMM's.  On a B200 this pays in short bursts (the 28672 x 8192 projection at 4096 rows: 1.50 ms per layer against
1.75 ms back to back over a 40 ms loop) and is neutral in a seconds-long loop, where the 1 kW power
limit, not the schedule, sets the pace.

Usage::

    ahead = DecodeAhead(layers_in_execution_order, dtype=torch.bfloat16)   # allocates two weight buffers
    ...                      # forwards as usual: layer i waits for its weight, then sends layer i+1's
    ahead.join()             # the current stream waits for the side stream (end of a pass / capture)
    ahead.close()

Layers are matched by identity; a layer that is called out of order simply decodes when it is
called (on the side stream, nothing overlapped) -- results never depend on the order.  Works
under CUDA-graph capture (the side stream forks from and joins the capturing stream through
events; call ``join()`` before the capture ends).  ``ShardedLinear`` wrappers are looked through.
"""

from __future__ import annotations

import torch

from .np_vq_linear import NPVQLinear

__all__ = ["DecodeAhead"]


def _inner(layer) -> NPVQLinear:
    local = getattr(layer, "local", layer)   # sharding.ShardedLinear keeps its shard in .local
    if not isinstance(local, NPVQLinear):
        raise TypeError(f"DecodeAhead takes NPVQLinear layers (or shards of them), got {type(local).__name__}.")
    return local


class DecodeAhead:
    """Two dense-weight buffers shared by ``layers`` and a side stream that fills them one layer
    ahead of the GEMMs.  ``layers``: the large-batch linears in the order the model calls them."""

    def __init__(self, layers, dtype: torch.dtype = torch.bfloat16) -> None:
        self.layers = [_inner(m) for m in layers]
        if not self.layers:
            raise ValueError("DecodeAhead needs at least one layer.")
        self.dtype = dtype
        dev = self.layers[0].packed_indices.device
        if dev.type != "cuda":
            raise RuntimeError("DecodeAhead needs layers on a CUDA device.")
        self.device = dev
        elems = max(m.out_features * m.in_features for m in self.layers)
        self._buf = [torch.empty(elems, dtype=dtype, device=dev) for _ in range(2)]
        self._side = torch.cuda.Stream(device=dev)
        self._index = {id(m): i for i, m in enumerate(self.layers)}
        self._holds: list[int | None] = [None, None]      # layer index whose weight each buffer holds / will hold
        self._filled = [torch.cuda.Event(), torch.cuda.Event()]   # recorded on the side stream after a decode
        self._freed = [torch.cuda.Event(), torch.cuda.Event()]    # recorded by the consumer after its GEMM
        self._used = [False, False]                        # whether _freed[b] has been recorded since the last fill
        self._next_buf = 0
        self.enabled = True          # False: layers decode by themselves, back to back with their GEMM
        self._dirty = False          # something was sent to the side stream since the last join()
        for m in self.layers:
            m._decode_ahead = self

    # ---- called by NPVQLinear._forward_dequant_gemm -------------------------------------------
    def weight_for(self, layer: NPVQLinear, dtype: torch.dtype) -> torch.Tensor | None:
        """The decoded weight of ``layer`` (``[N, K]`` of ``dtype``), valid on the current stream;
        also sends the decode of the layer after it.  None: not one of this object's layers or
        another dtype (the caller decodes by itself)."""
        i = self._index.get(id(layer))
        if i is None or dtype != self.dtype or not self.enabled:
            return None
        cur = torch.cuda.current_stream(self.device)
        b = self._holds.index(i) if i in self._holds else self._issue(i, cur)
        cur.wait_event(self._filled[b])
        if i + 1 < len(self.layers) and (i + 1) not in self._holds:
            self._issue(i + 1, cur, keep=b)
        m = self.layers[i]
        return self._buf[b][: m.out_features * m.in_features].view(m.out_features, m.in_features)

    def release(self, layer: NPVQLinear) -> None:
        """After the GEMM that read ``layer``'s weight was launched on the current stream."""
        i = self._index.get(id(layer))
        if i is None or i not in self._holds:
            return
        b = self._holds.index(i)
        self._freed[b].record(torch.cuda.current_stream(self.device))
        self._used[b] = True
        self._holds[b] = None

    # ---- user side --------------------------------------------------------------------------------
    def join(self) -> None:
        """The current stream waits for everything sent to the side stream; decoded weights that
        were not consumed are dropped."""
        if self._dirty:
            ev = torch.cuda.Event()
            ev.record(self._side)
            torch.cuda.current_stream(self.device).wait_event(ev)
            self._dirty = False
        self._holds = [None, None]
        self._used = [False, False]

    def close(self) -> None:
        self.join()
        for m in self.layers:
            if getattr(m, "_decode_ahead", None) is self:
                m._decode_ahead = None
        self._buf = []

    # ---- internals --------------------------------------------------------------------------------
    def _issue(self, i: int, cur: torch.cuda.Stream, keep: int | None = None) -> int:
        """Decode layer i on the side stream into a buffer other than ``keep``."""
        b = 1 - keep if keep is not None else self._next_buf
        self._next_buf = 1 - b
        self._dirty = True
        fork = torch.cuda.Event()
        fork.record(cur)
        self._side.wait_event(fork)            # not before the caller's point in its stream ...
        if self._used[b]:
            self._side.wait_event(self._freed[b])   # ... nor before the buffer's last reader is done
            self._used[b] = False
        m = self.layers[i]
        out = self._buf[b][: m.out_features * m.in_features].view(m.out_features, m.in_features)
        with torch.cuda.stream(self._side):
            m._decode_dense(self.dtype, out)
            self._filled[b].record(self._side)
        self._holds[b] = i
        return b
