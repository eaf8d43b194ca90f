"""A layer: norm -> mixers in parallel on the same normed input -> residual; norm ->
feed-forward -> residual.  A feed-forward without a norm of its own reads the mixers' normed input
and is one more parallel summand.  With output norms (LayerSpec.mixer_out_norm, ffn_out_norm) a sublayer's
result is collected in a 32-bit buffer of its own, normed, and then added.

CodeClaper/tinyllama.c falcon_h1.c:311-395: n = norm(x); x = (x + attn(n)) + ssm(n);
x = x + ffn(norm(x)).  The residual stream is 32-bit; each mixer and the feed-forward add
their output into it in the order they are listed.
"""
from __future__ import annotations

import inspect
import os
from typing import Dict, List, Optional

import torch

from .base import LayerCache, LayerSpec, Part, StepInfo, WeightSpec, act_empty, scratch_buf, scratch_is_shared
from .linear import StackedLinear


# Mixers that are independent of one another between their input and output projections run side by side on
# streams of their own.  One-token steps are chains of short kernels; in a prompt the walk over a sequence's chunks
# keeps a block on two SMs in three for most of its time, and the attention kernel's blocks, one to an SM, take the
# rest (2,048 tokens: 9.71 -> 9.31 ms).  TLC_PARALLEL_PROMPT_MIXERS=0 keeps prompts on one stream.
PARALLEL_MIXERS = bool(int(os.environ.get("TLC_PARALLEL_MIXERS", "1")))
_MAIN_MIXER = int(os.environ["TLC_MAIN_MIXER"]) if "TLC_MAIN_MIXER" in os.environ else None
FUSE_OUTPUTS = bool(int(os.environ.get("TLC_FUSE_OUTPUTS", "1")))
PARALLEL_PROMPT_MIXERS = bool(int(os.environ.get("TLC_PARALLEL_PROMPT_MIXERS", "1")))
# In a prompt the mixers' long kernels want an SM for each of their blocks.  One of a side stream that is resident
# first keeps the current stream's blocks waiting until its own have finished; a side mixer that can
# (mix_takes_max_blocks) may be told to hold at most this many SMs and to work through its tiles with them.
# 0: no bound, the default.  Measured at the 1.5B sizes (2,048 tokens; the walk over the chunks has 96 blocks,
# attention 128): with 48 the walk ends 12 us earlier (86 -> 143.5 us after the layer's start instead of 155.7),
# attention takes 53 us instead of 30, and the part of the scan that runs beside both finds no room and ends
# as late as the walk did before: 7.51 ms a step either way.  The three kernels fill the SMs between them.
PROMPT_SIDE_BLOCKS = int(os.environ.get("TLC_PROMPT_SIDE_BLOCKS", "0"))
# A feed-forward that runs beside the mixers on their normed input (a parallel layer) and can hand over its terms
# (forward_parts / add_parts): in one-token steps the two are chains of short kernels and run on two streams; the terms are
# added into the residual stream after the mixers' outputs, on the current stream, so the order of the sums is fixed.
# TLC_PARALLEL_FFN=1 (the default) puts the MIXERS on a side stream of high priority and the feed-forward on the current
# one, 2 the feed-forward on the side stream, 0 runs it after the mixers.  Measured with four layers of experts beside
# latent attention, attention and a delta rule at width 2048: a step at batch 8 0.654 ms (0), 0.577 (2), 0.543 (1); at
# batch 64 0.957, 0.857, 0.864.  A prompt of 2,048 tokens gains nothing (3.89 ms one after the other, 3.95 and 4.09 side
# by side: the experts' products fill the GPU by themselves and slow the mixers' kernels beside them), so prompts run
# one after the other unless TLC_PARALLEL_FFN_PROMPTS=1.
PARALLEL_FFN = int(os.environ.get("TLC_PARALLEL_FFN", "1"))
PARALLEL_FFN_PROMPTS = bool(int(os.environ.get("TLC_PARALLEL_FFN_PROMPTS", "0")))


_streams = {}


def _current_stream(device) -> "torch.cuda.Stream":
    """The current stream of the device as a torch object.  torch.cuda.current_stream() takes some 10 us of Python
    a call and a block asks once a layer, so the object is kept by the stream's handle (which torch's raw query
    gives in a fraction of that) and made anew only when the handle is a new one."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is None:
        return torch.cuda.current_stream(index)
    handle = raw(index)
    hit = _streams.get((index, handle))
    if hit is None:
        if len(_streams) > 64:
            _streams.clear()
        hit = _streams[(index, handle)] = torch.cuda.current_stream(index)
    return hit


class Block(Part):
    def __init__(self, spec: LayerSpec, act_dtype_of=None):
        self.spec = spec
        self.mixer_norm = spec.mixer_norm.build()
        self.mixers = [m.build() for m in spec.mixers]
        self.ffn_norm = spec.ffn_norm.build() if spec.ffn_norm is not None else None
        self.ffn = spec.ffn.build() if spec.ffn is not None else None
        self.mixer_out_norm = spec.mixer_out_norm.build() if spec.mixer_out_norm is not None else None
        self.ffn_out_norm = spec.ffn_out_norm.build() if spec.ffn_out_norm is not None else None
        # how the mixers' results are joined where that is not their sum (each normed by itself, then averaged)
        self.mixer_join = spec.mixer_join.build() if spec.mixer_join is not None else None
        if self.mixer_join is not None and not self.mixers:
            raise ValueError("a join of the mixers' results needs mixers")
        # a feed-forward without a norm of its own is a parallel branch: it reads the mixers' normed input; so is one
        # whose own norm is applied to the layer's input (LayerSpec.parallel)
        self.parallel_ffn = self.ffn is not None and (self.ffn_norm is None or bool(spec.parallel))
        self.own_parallel_norm = self.parallel_ffn and self.ffn_norm is not None
        if self.parallel_ffn and (not self.mixers or self.ffn_out_norm is not None or self.mixer_out_norm is not None):
            raise ValueError("a feed-forward without a norm of its own runs beside the mixers on their normed input: the layer "
                             "needs mixers and takes no output norms")
        self.dtype: Optional[torch.dtype] = None
        # a part whose forward() takes `accumulate` can overwrite its target instead of adding into it
        takes = lambda p: p is not None and "accumulate" in inspect.signature(p.forward).parameters
        self._mixer_overwrites = [takes(m) for m in self.mixers]
        self._ffn_overwrites = takes(self.ffn)

    def parts(self) -> List[Part]:
        return [p for p in [self.mixer_norm, *self.mixers, self.mixer_join, self.mixer_out_norm, self.ffn_norm, self.ffn,
                            self.ffn_out_norm] if p is not None]

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def cache_requests(self) -> list:
        return [r for p in self.parts() for r in p.cache_requests()]

    def step_requests(self) -> list:
        return [r for p in self.parts() for r in p.step_requests()]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.dtype = dtype
        for p in self.parts():
            p.bind(tensors, dtype, device)
        # Mixers that run in parallel on the same normed input and say what they first project it to
        # share one product: their input projections are stacked.  Any other mixer gets the normed
        # input as a tensor.
        self.fused_in, self.fused_offsets = None, []
        if len(self.mixers) > 1 and (self.mixer_out_norm is None or self.mixer_join is not None) \
                and all(hasattr(m, "input_projection") and hasattr(m, "forward_projected")
                                        for m in self.mixers):
            projs = [m.input_projection() for m in self.mixers]
            self.fused_in = StackedLinear.fuse_bound(projs)
            off = 0
            for pr in projs:
                self.fused_offsets.append((off, pr.out_features))
                off += pr.out_features
        # Likewise their output projections, whose results are added into the residual stream: the mixers
        # write side by side into one buffer, and one product over the weights side by side along K forms
        # the sum in its accumulator.
        self.fused_out, self.out_offsets, self.out_scales = None, [], []
        if self.fused_in is not None and self.mixer_join is None and FUSE_OUTPUTS and all(hasattr(m, "output_projection") and hasattr(m, "mix")
                                                              for m in self.mixers):
            outs = [m.output_projection() for m in self.mixers]
            fused = StackedLinear.fuse_bound_inputs(outs, [bool(getattr(m, "mix_takes_scale", False)) for m in self.mixers])
            if fused is not None:
                self.fused_out, self.out_scales = fused
                off = 0
                for pr in outs:
                    self.out_offsets.append((off, pr.in_features))
                    off += pr.in_features

    def _mix_in_parallel(self, parts, step: StepInfo, cache: LayerCache, x32: torch.Tensor, outs: Optional[torch.Tensor] = None) -> None:
        """One mixer runs on the current stream, every other on a side stream that starts after the
        shared input projection.  Output projections add into the residual stream one after the
        other on the current stream, in the mixers' order, each after its mixer has finished.  (Under stream capture the
        side streams become parallel branches of the graph.)  outs [T, n, D]: every mixer's output projection is written
        to its own rows outs[:, i] instead (a layer that joins its mixers' results by something else than their sum)."""
        main = _current_stream(x32.device)
        if not hasattr(self, "_side"):
            self._side = [torch.cuda.Stream(device=x32.device) for _ in self.mixers[1:]]
            # events are made once: a record overwrites the event's last state, and every wait of this block follows
            # its record in program order
            self._fork = torch.cuda.Event()
            self._done = [torch.cuda.Event() for _ in self.mixers]
        # the mixer with the longest chain of kernels stays on the current stream, where every
        # kernel follows its predecessor by a programmatic edge
        lengths = [int(getattr(m, "single_token_launches", 1)) for m in self.mixers]
        here = _MAIN_MIXER if _MAIN_MIXER is not None else lengths.index(max(lengths))
        fork = self._fork
        fork.record(main)
        acts, done = [None] * len(self.mixers), [None] * len(self.mixers)
        joint, views = self._joint_activations(x32)
        sides = iter(self._side)
        for i, (m, part) in enumerate(zip(self.mixers, parts)):
            if i == here:
                continue
            side = next(sides)
            side.wait_event(fork)
            torch.cuda.set_stream(side)              # (the context manager asks for the current stream again: 10 us)
            try:
                bound = PROMPT_SIDE_BLOCKS if step.max_new > 1 and getattr(m, "mix_takes_max_blocks", False) else 0
                acts[i] = self._mix(i, part, step, cache, views[i], max_blocks=bound)
                done[i] = self._done[i]
                done[i].record(side)
            finally:
                torch.cuda.set_stream(main)
        # The wait for the side streams breaks the chain of programmatic launches on this stream.  A mixer that
        # offers to (mix_takes_join) places it before its own last kernel; otherwise it comes after the mixer.
        joined = []

        def join():
            if not joined:
                joined.append(True)
                for ev in done:
                    if ev is not None:
                        main.wait_event(ev)

        early = getattr(self.mixers[here], "mix_takes_join", False)
        acts[here] = self._mix(here, parts[here], step, cache, views[here], join if early else None)
        join()
        for i, m in enumerate(self.mixers):          # outputs in the mixers' order, whatever ran where
            if outs is not None:
                m.output_projection().forward(acts[i], outs[:, i], accumulate=False)
            elif joint is None:
                m.output(acts[i], x32)
        if joint is not None:
            self.fused_out.forward(joint, x32, accumulate=True)

    def _mix(self, i: int, part: torch.Tensor, step: StepInfo, cache: LayerCache, view: Optional[torch.Tensor], join=None,
             max_blocks: int = 0):
        """Mixer i between its projections; into its columns of the joint buffer, scaled, where there is one."""
        m = self.mixers[i]
        more = {} if join is None else {"join": join}
        if max_blocks:
            more["max_blocks"] = max_blocks
        if view is None:
            return m.mix(part, step, cache, **more)
        if self.out_scales[i] != 1.0:
            return m.mix(part, step, cache, view, self.out_scales[i], **more)
        return m.mix(part, step, cache, view, **more)

    def _joint_activations(self, x32: torch.Tensor):
        """The buffer that the mixers fill side by side for the shared output projection, and each
        mixer's columns of it; (None, Nones) without a shared output projection."""
        if self.fused_out is None:
            return None, [None] * len(self.mixers)
        joint = scratch_buf("block.joint", (x32.shape[0], self.fused_out.in_features), self.dtype, x32.device)
        return joint, [joint[:, off:off + n] for off, n in self.out_offsets]

    def _beside(self, x32: torch.Tensor, step: StepInfo):
        """Whether this layer's feed-forward runs beside its mixers on two streams in this step."""
        return bool(self.parallel_ffn and PARALLEL_FFN and x32.is_cuda and (step.max_new == 1 or PARALLEL_FFN_PROMPTS)
                    and hasattr(self.ffn, "forward_parts") and hasattr(self.ffn, "add_parts"))

    def _parallel_inputs(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache):
        """(what the mixers read, what a parallel feed-forward reads): one normed copy of the layer's input, or, where the
        feed-forward has a norm of its own, two; norms that share their statistics (pairs_with) make both in one kernel."""
        if not self.own_parallel_norm:
            normed = self._pre_norm(self.mixer_norm, x32, "block.normed", step, cache)
            return normed, normed
        pairs = getattr(self.mixer_norm, "pairs_with", None)
        if pairs is not None and pairs(self.ffn_norm):
            normed = scratch_buf("block.normed", x32.shape, self.dtype, x32.device)
            ffn_in = scratch_buf("block.ffn_normed", x32.shape, self.dtype, x32.device)
            self.mixer_norm.forward_pair(x32, normed, self.ffn_norm, ffn_in)
            return normed, ffn_in
        return (self._pre_norm(self.mixer_norm, x32, "block.normed", step, cache),
                self._pre_norm(self.ffn_norm, x32, "block.ffn_normed", step, cache))

    def _two_branches(self, normed: torch.Tensor, x32: torch.Tensor, run_mixers, ffn_in: Optional[torch.Tensor] = None) -> None:
        """A parallel layer on two streams (under stream capture: two branches of the graph): the mixers, which add
        their outputs into the residual stream, and the feed-forward's terms; the terms are added after the branches have
        met, on the current stream, so the order of the sums is fixed.  run_mixers(): launches the mixers on whatever
        stream is current."""
        main = _current_stream(x32.device)
        if not hasattr(self, "_ffn_side"):
            least, greatest = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
            self._ffn_side = torch.cuda.Stream(device=x32.device, priority=greatest if PARALLEL_FFN == 1 else least)
            self._ffn_fork, self._ffn_done = torch.cuda.Event(), torch.cuda.Event()
        side = self._ffn_side
        self._ffn_fork.record(main)                   # after the norm whose output both branches read
        side.wait_event(self._ffn_fork)
        terms = None
        torch.cuda.set_stream(side)
        try:
            if PARALLEL_FFN == 1:
                run_mixers()
            else:
                terms = self.ffn.forward_parts(normed if ffn_in is None else ffn_in)
            self._ffn_done.record(side)
        finally:
            torch.cuda.set_stream(main)
        if PARALLEL_FFN == 1:
            terms = self.ffn.forward_parts(normed if ffn_in is None else ffn_in)
        else:
            run_mixers()
        main.wait_event(self._ffn_done)
        self.ffn.add_parts(terms, x32)

    def _joined_mixers(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache, copy: Optional[torch.Tensor] = None) -> None:
        """x <- x + out_norm(join(mixer_i(h))): every mixer's result in rows of its own, then the join (and the norm after
        it) in one kernel.  Mixers that offer their projections share the input product and, in one-token steps, run side
        by side on streams."""
        reads = [bool(getattr(m, "reads_stream", False)) and getattr(self.mixer_norm, "identity", False) for m in self.mixers]
        normed = None if all(reads) else self._pre_norm(self.mixer_norm, x32, "block.normed", step, cache)
        T, n = x32.shape[0], len(self.mixers)
        outs = scratch_buf("block.joined", (T, n, x32.shape[1]), torch.float32, x32.device)
        if self.fused_in is not None and all(hasattr(m, "mix") and hasattr(m, "output_projection") for m in self.mixers):
            proj = scratch_buf("block.proj", (T, self.fused_in.out_features), torch.float32, x32.device)
            self.fused_in.forward(normed, proj)
            parts = [proj[:, off:off + w] for off, w in self.fused_offsets]
            if (step.max_new == 1 or PARALLEL_PROMPT_MIXERS) and x32.is_cuda and PARALLEL_MIXERS:
                self._mix_in_parallel(parts, step, cache, x32, outs)
            else:
                for i, (m, part) in enumerate(zip(self.mixers, parts)):
                    m.output_projection().forward(m.mix(part, step, cache), outs[:, i], accumulate=False)
        else:
            for i, m in enumerate(self.mixers):
                if not self._mixer_overwrites[i]:
                    raise ValueError("a layer that joins its mixers' results needs mixers whose forward() can overwrite its target")
                m.forward(x32 if reads[i] else normed, step, cache, outs[:, i], accumulate=False)
        self.mixer_join.add_joined(outs, x32, self.mixer_out_norm, copy=copy)

    # A sublayer without a norm in front reads the residual stream in the activation type.  The kernel that last added
    # into the stream (an output norm) writes that copy as its second output, so that no kernel of its own has to make it:
    # _stream_copy() names the buffer to the adding kernel and notes that it is filled, _pre_norm() then hands it over.
    @property
    def reads_stream_copy(self) -> bool:
        """Whether this layer's first step is a copy of the residual stream in the activation type (no norm before the
        mixers, and a mixer that does not take the 32-bit rows themselves)."""
        return bool(self.mixers) and self._plain_copy(self.mixer_norm) \
            and not all(bool(getattr(m, "reads_stream", False)) for m in self.mixers)

    @staticmethod
    def _plain_copy(norm) -> bool:
        return norm is not None and getattr(norm, "identity", False) and not hasattr(norm, "forward_step")

    def _stream_copy(self, tag: str, x32: torch.Tensor) -> Optional[torch.Tensor]:
        if not (x32.is_cuda and scratch_is_shared()):
            return None
        self._copied.add(tag)
        return scratch_buf(tag, x32.shape, self.dtype, x32.device)

    def _pre_norm(self, norm, x32: torch.Tensor, tag: str, step: StepInfo, cache: LayerCache) -> torch.Tensor:
        normed = scratch_buf(tag, x32.shape, self.dtype, x32.device)
        if tag in self._copied:                       # filled by the kernel that last added into the stream
            self._copied.discard(tag)
            return normed
        if hasattr(norm, "forward_step"):             # a norm with per-sequence state (token shift)
            norm.forward_step(x32, normed, step, cache)
        else:
            norm.forward(x32, normed)
        return normed

    def forward(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache, copy_ready: bool = False,
                copy_for_next: bool = False) -> bool:
        """Updates the float32 residual stream x32 [T, D] in place.  copy_ready: the layer before has left the stream in
        the activation type where this layer's mixers look for it; copy_for_next: the next layer wants the same of this
        one.  Returns whether that copy was written."""
        self._copied = {"block.normed"} if copy_ready and self.reads_stream_copy and scratch_is_shared() else set()
        last_add_is_mixers = self.ffn is None or self.parallel_ffn
        copy = None
        if self.mixers and self.mixer_out_norm is not None:
            if last_add_is_mixers:
                copy = self._stream_copy("block.normed", x32) if copy_for_next and self.ffn is None else None
            elif self._plain_copy(self.ffn_norm):
                copy = self._stream_copy("block.ffn_normed", x32)
        if self.mixers and self.mixer_join is not None:
            self._joined_mixers(x32, step, cache, copy)
        elif self.mixers and self.mixer_out_norm is not None:
            # x <- x + out_norm(sum of the mixers' outputs); a mixer that reads the stream itself gets the 32-bit rows
            reads = [bool(getattr(m, "reads_stream", False)) and getattr(self.mixer_norm, "identity", False) for m in self.mixers]
            normed = None if all(reads) else self._pre_norm(self.mixer_norm, x32, "block.normed", step, cache)
            y = scratch_buf("block.mixed", x32.shape, torch.float32, x32.device)
            if not self._mixer_overwrites[0]:
                y.zero_()
            for i, m in enumerate(self.mixers):
                if self._mixer_overwrites[i]:
                    m.forward(x32 if reads[i] else normed, step, cache, y, accumulate=i > 0)
                else:
                    m.forward(x32 if reads[i] else normed, step, cache, y)
            self.mixer_out_norm.add_normed(y, x32, copy=copy)
        elif self.mixers:
            normed, ffn_in = self._parallel_inputs(x32, step, cache) if self.parallel_ffn \
                else (self._pre_norm(self.mixer_norm, x32, "block.normed", step, cache), None)
            if self._beside(x32, step):
                self._two_branches(normed, x32, lambda: self._run_mixers(normed, x32, step, cache), ffn_in)
                return False
            self._run_mixers(normed, x32, step, cache)
        if self.parallel_ffn:
            # h was normed before the mixers added anything; the sum x + mixers(h) + ffn(h) forms in the residual stream
            self.ffn.forward(ffn_in, x32)
            return False
        if self.ffn is not None:
            return self._feed_forward(x32, step, cache, copy_for_next)
        return copy is not None

    def _run_mixers(self, normed: torch.Tensor, x32: torch.Tensor, step: StepInfo, cache: LayerCache) -> None:
        """The mixers of a layer without a mixer output norm, from their shared normed input into the residual stream."""
        if self.fused_in is not None:
            proj = scratch_buf("block.proj", (x32.shape[0], self.fused_in.out_features), torch.float32, x32.device)
            self.fused_in.forward(normed, proj)
            parts = [proj[:, off:off + n] for off, n in self.fused_offsets]
            if (step.max_new == 1 or PARALLEL_PROMPT_MIXERS) and x32.is_cuda and PARALLEL_MIXERS and all(hasattr(m, "mix") for m in self.mixers):
                self._mix_in_parallel(parts, step, cache, x32)
            elif self.fused_out is not None:
                joint, views = self._joint_activations(x32)
                for i, (part, view) in enumerate(zip(parts, views)):
                    self._mix(i, part, step, cache, view)
                self.fused_out.forward(joint, x32, accumulate=True)
            else:
                for m, part in zip(self.mixers, parts):
                    m.forward_projected(part, step, cache, x32)
        else:
            for m in self.mixers:
                m.forward(normed, step, cache, x32)

    def _feed_forward(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache, copy_for_next: bool = False) -> bool:
        """A feed-forward with a norm of its own, after the mixers.  Returns whether the kernel that added its result
        also left the stream in the activation type for the next layer (copy_for_next)."""
        normed = self._pre_norm(self.ffn_norm, x32, "block.ffn_normed", step, cache)
        copy = self._stream_copy("block.normed", x32) if copy_for_next and self.ffn_out_norm is not None else None
        self._copied.discard("block.normed")          # (the next layer is told by the return value)
        # without a norm in front, a feed-forward that can use them (takes_stream) also gets the 32-bit rows themselves
        more = {"stream": x32} if getattr(self.ffn_norm, "identity", False) and getattr(self.ffn, "takes_stream", False) else {}
        if self.ffn_out_norm is None:
            self.ffn.forward(normed, x32, **more)
        elif hasattr(self.ffn, "forward_parts"):
            # a feed-forward whose result is a sum of terms hands them to the norm, which adds them up itself
            parts, extra, gate = self.ffn.forward_parts(normed, **more)
            self.ffn_out_norm.add_normed(parts, x32, extra, gate, copy=copy)
        else:
            y = scratch_buf("block.ffn_out", x32.shape, torch.float32, x32.device)
            if self._ffn_overwrites:
                self.ffn.forward(normed, y, accumulate=False)
            else:
                y.zero_()
                self.ffn.forward(normed, y)
            self.ffn_out_norm.add_normed(y, x32, copy=copy)
        return copy is not None
