"""The engine: a model, its cache and ONE step function.

``step`` takes a batch of sequences, each with its next tokens (a whole prompt, or one token, or any run in
between) and the places whose logits are wanted. It runs only those tokens, as one packed batch, against the cache
that earlier steps left, stores their keys and values, and returns 32-bit logits at the wanted places. Sequences
are never padded to one another's length (the only padding are whole rows at the end of a recorded short prompt
step, which belong to no sequence and store nothing), so no result depends on padding. In float32 a row's logits do not depend on what else is in the batch or
on how the tokens were cut into steps, bit for bit: every sum is taken in an order that depends on positions only.
In bfloat16 they agree up to rounding: the serving kernels choose tile widths and the number of ways a product or a
sequence's keys are split from the step's row count, so the last bits - and with them a greedy token at a near tie -
can differ with the batch.

The reference has three entry points for one sequence - ``step`` (one token, ``kindi/nanbeige.py:736-776``),
``prefill_batch`` (a prompt in chunks, head on the last row, ``:962-1021``) and ``check`` (up to 8 rows with logits
for each, ``:1144-1192``); this one function covers all three for a batch.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..cache.pages import CacheFull
from ..cache.sequence_cache import SequenceCache
from ..config.registry import model_from_dir
from ..config.spec import ModelSpec
from ..kernels import lib as K
from ..parts.base import StepContext
from ..parts.model import DecoderModel, cache_needs, expected_tensors
from ..weights.loader import load_tensors
from .batch import PackedStep, StepEntry, pack, split_step

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
from ..config.runtime import GREEDY as _GREEDY      # noqa: E402


class EngineError(RuntimeError):
    pass


class OutOfDeviceMemory(EngineError):
    """the weights, the cache and the working memory of the largest step do not fit the GPU's free memory"""


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, ctx: int = 24576, dtype: str = "bfloat16",
                 max_batch: int = 64, device: str = "cuda:0", spec: Optional[ModelSpec] = None,
                 tensors: Optional[Mapping[str, torch.Tensor]] = None, cuda_graphs: bool = True,
                 max_step_tokens: int = 8192, prompt_graph_tokens: int = 512, log=None):
        """``model_dir``: a folder with config.json and safetensors files; or give ``spec`` and ``tensors``
        directly. ``ctx``: the most tokens all live sequences hold together (rounded up per sequence to the cache
        page); it sizes the cache, like the reference's ``ctx`` (``kindi/nanbeige.py:245``). ``prompt_graph_tokens``:
        prompt steps of up to this many tokens are recorded too, padded to a multiple of 64 rows (0: never)."""
        if dtype not in _DTYPES:
            raise EngineError("dtype must be 'bfloat16' or 'float32', not %r" % (dtype,))
        if not torch.cuda.is_available():
            raise EngineError("kindi_b200 runs on a CUDA GPU only (sm_100a); none is visible")
        self.log = log or (lambda msg: None)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        K.load()                                   # build / load the kernels now: fail loudly, not at first step
        self.dtype_name = dtype
        self.dtype = _DTYPES[dtype]
        self.config = None                         # the architecture's typed configuration (None with ``spec=``)
        if spec is None:
            if model_dir is None:
                raise EngineError("give a model folder, or a spec with tensors")
            # the folder's architecture name picks the registry entry, which reads its own config.json keys
            self.config, spec = model_from_dir(model_dir)
        self.spec = spec
        self.ctx = int(ctx)
        self.max_batch = int(max_batch)
        self.max_step_tokens = max(64, int(max_step_tokens))     # longer steps are run in pieces of this many tokens
        self.prompt_graph_tokens = max(0, int(prompt_graph_tokens)) if cuda_graphs else 0
        self.prompt_graphs_kept = 12                   # the most recorded prompt shapes kept (each holds its buffers)
        self.plan = self._plan_memory(spec, tensors)
        if tensors is None:
            tensors = load_tensors(model_dir, expected_tensors(spec), run_dtype=dtype, device=str(self.device),
                                   may_ignore=spec.may_ignore, copies=spec.copies, log=self.log)
        else:
            tensors = {n: _to_run_dtype(t, dtype).to(self.device) for n, t in tensors.items()}
        self.model = DecoderModel(spec, tensors, dtype=self.dtype, device=self.device)
        self.cache = SequenceCache(cache_needs(spec), max_tokens=self.ctx, n_slots=self.max_batch,
                                   dtype=self.dtype, device=self.device, max_step_tokens=self.max_step_tokens)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the tokens picked by the latest step, in the order of its wanted rows: a later step can take its tokens from
        # here on the device, so the host need not have read them before it issues that step
        self._picked = torch.zeros(max(self.max_batch, 1), dtype=torch.int32, device=self.device)
        self._pinned: Dict[int, torch.Tensor] = {}
        self.steps_run = 0
        self.cuda_graphs = bool(cuda_graphs) and self.model.graph_safe
        self._graphs: Dict[tuple, "_StepGraph"] = {}
        self.graph_replays = 0
        self._graph_warm = set()

    def _plan_memory(self, spec: ModelSpec, tensors) -> Dict[str, int]:
        """what the engine will hold on the device, counted before anything is allocated: the weights (twice the
        fused ones while a part joins them), the cache, and the activations of the largest step; more than the GPU
        has free is an error here, not an out-of-memory fault in the middle of loading. The reference plans its
        memory before it loads in the same way (``kindi/nanbeige.py:316-397``)."""
        el = 4 if self.dtype == torch.float32 else 2
        shapes = expected_tensors(spec)
        weights = 0
        if tensors is None or any(not t.is_cuda for t in tensors.values()):
            for n, shape in shapes.items():
                k = 1
                for d in shape:
                    k *= d
                weights += k * el
        cache = SequenceCache.bytes_needed(cache_needs(spec), self.ctx, self.max_batch, self.dtype,
                                           self.max_step_tokens)
        widest = max([spec.width] + [s[0] for s in shapes.values() if len(s) == 2 and s[0] != spec.vocab_size])
        rows = min(self.max_step_tokens, self.ctx)
        # residual + branch planes in 32-bit, the widest activation twice in the run dtype, logits of a decode batch;
        # every recorded prompt shape keeps buffers of its own for its rows
        per_row = 3 * spec.width * 4 + 2 * widest * max(el, 2)
        work = (rows + self.prompt_graphs_kept * self.prompt_graph_tokens) * per_row \
            + self.max_batch * spec.vocab_size * 4 * 2
        plan = {"weights": weights, "cache": cache, "work": work, "total": weights + cache + work}
        free, total = torch.cuda.mem_get_info(self.device)
        plan["free"] = int(free)
        gib = 2.0 ** 30
        self.log("memory plan: weights %.2f GiB, cache %.2f GiB (ctx %d, %d slots), working memory of a %d-token step "
                 "%.2f GiB; %.2f of %.2f GiB free on %s" % (weights / gib, cache / gib, self.ctx, self.max_batch, rows,
                                                            work / gib, free / gib, total / gib, self.device))
        if plan["total"] > free:
            raise OutOfDeviceMemory(
                "the model does not fit: weights %.2f GiB + cache %.2f GiB (ctx %d tokens, %d slots) + working memory "
                "%.2f GiB = %.2f GiB, and %s has %.2f GiB free; lower ctx (the cache grows with it), max_batch or "
                "max_step_tokens" % (weights / gib, cache / gib, self.ctx, self.max_batch, work / gib,
                                     plan["total"] / gib, self.device, free / gib))
        return plan

    # ------------------------------------------------------------------ slots
    def alloc(self) -> int:
        """take a slot for a sequence that starts"""
        return self.cache.alloc_slot()

    def free(self, slot: int) -> None:
        """give back a sequence's slot and everything it holds"""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], greedy: bool = False, tokens_from_previous: bool = False):
        """run the entries' tokens as one batch; returns float32 logits ``[number of wanted places, vocab]`` on the
        device (None when nothing is wanted). The cache then holds the tokens' keys and values. With ``greedy`` the
        return value is ``(logits, tokens)``, ``tokens`` being the argmax of each wanted row (int32, on the device;
        in the recorded decode step the pick is part of the recording). The tensors belong to the engine until its
        next step.

        ``tokens_from_previous`` (a step of one token per sequence only): entry i's token is the one the previous
        step picked for its i-th wanted row (``pick`` or ``greedy``), taken on the device; the entries' own token
        values are ignored. The host can then issue this step before it has read the previous step's tokens (the
        reference overlaps host and GPU the same way: ``step_begin`` / ``step_end``, ``kindi/nanbeige.py:741-776``)."""
        if tokens_from_previous and (any(len(e.tokens) != 1 for e in entries) or len(entries) > self._picked.numel()):
            raise ValueError("tokens_from_previous needs a step of one token per sequence")
        if sum(len(e.tokens) for e in entries) > self.max_step_tokens:
            return self._step_in_pieces(entries, greedy)
        cache = self.cache
        before = [cache.length[e.slot] for e in entries]
        limit = self.spec.max_positions
        if limit is not None:
            for e, n in zip(entries, before):
                if n + len(e.tokens) > limit:
                    raise EngineError("the sequence in slot %d would reach %d positions; the model's configuration "
                                      "allows %d (max_position_embeddings)" % (e.slot, n + len(e.tokens), limit))
        # Recorded steps. The steady decode shape (one token and one wanted row per sequence) is recorded once per
        # batch size and replayed (the reference records one graph per token too, kindi/nanbeige.py:728-734). Short
        # prompt steps are bound by the host's launch-by-launch issue, not by the GPU: they are padded to a multiple
        # of 64 rows and recorded per (rows, sequences, wanted rows). Lengths, slots, row ranges and tokens are read
        # from device memory by the kernels, so a recording serves every step of its shape.
        n_tok = sum(len(e.tokens) for e in entries)
        key = None
        if self.cuda_graphs:
            if n_tok == len(entries):
                if all(e.want == (0,) for e in entries):
                    key = ("decode", len(entries))
            elif n_tok <= self.prompt_graph_tokens and not tokens_from_previous:
                key = ("prompt", (n_tok + 63) // 64 * 64, len(entries), sum(len(e.want) for e in entries))
        ps = pack(entries, before, pad_rows_to=key[1] if key and key[0] == "prompt" else 0)
        reserved = []
        try:
            for e, new_len in zip(entries, ps.h_kv_len):
                cache.reserve(e.slot, new_len)
                reserved.append(e.slot)
        except CacheFull as ex:
            raise CacheFull("%s while storing %d new tokens; the cache holds %d tokens (ctx = %d)"
                            % (ex, n_tok, cache.tokens_held(), self.ctx)) from None
        cache.flush()
        graph = None
        if key is not None:
            graph = self._graphs.get(key)
            if graph is None and key in self._graph_warm:
                if key[0] == "prompt":
                    kept = [k for k in self._graphs if k[0] == "prompt"]
                    if len(kept) >= self.prompt_graphs_kept:
                        del self._graphs[kept[0]]              # the oldest recorded prompt shape makes room
                graph = self._graphs[key] = _StepGraph(self, ps)
            self._graph_warm.add(key)
            if graph is None and ps.T != n_tok:
                ps = pack(entries, before)                     # not recorded (yet): run it without the padding rows
        picked = None
        if graph is not None:
            logits = graph.replay(ps, tokens_from_previous)
            picked = graph.picked
            self.graph_replays += 1
        else:
            ctx = self._context(ps)
            if tokens_from_previous:
                a, n = ps.off["tok"]
                self._meta_dev[a:a + n].copy_(self._picked[:n])
            rows = None
            if ps.R:
                a, n = ps.off["rows"]
                rows = self._meta_dev[a:a + n]
            logits = self.model.forward(ctx, rows)
        for e, new_len in zip(entries, ps.h_kv_len):
            cache.commit(e.slot, new_len)
        self.steps_run += 1
        if greedy:
            if picked is None and logits is not None:
                picked = self.pick(logits, _GREEDY)
            return logits, picked
        return logits

    def pick(self, logits: torch.Tensor, params, uniforms=None, histories=None) -> torch.Tensor:
        """the next token of each row of ``logits`` (the sampler's ``pick``), kept where a following step can take
        its tokens from (``tokens_from_previous``)"""
        R = logits.shape[0]
        out = self._picked[:R] if R <= self._picked.numel() else None
        return self._sampler().pick(logits, params, uniforms, histories, out=out)

    def _step_in_pieces(self, entries: Sequence[StepEntry], greedy: bool):
        """a step of more than max_step_tokens tokens: its pieces run one after another (activations stay bounded;
        a later piece reads the earlier ones from the cache) and the wanted rows are put back in the order of the
        entries and of their ``want`` lists"""
        for e in entries:
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError("want place %d lies outside the sequence's %d tokens of this step"
                                     % (w, len(e.tokens)))
        pieces = split_step(entries, self.max_step_tokens)
        got: Dict[Tuple[int, int], torch.Tensor] = {}            # (entry, place) -> logits row
        offset = [0] * len(entries)
        for sub in pieces:
            logits = self.step([e for _, e in sub])
            row = 0
            for i, e in sub:
                for w in e.want:
                    got[(i, offset[i] + w)] = logits[row].clone()
                    row += 1
                offset[i] += len(e.tokens)
        order = [(i, w) for i, e in enumerate(entries) for w in e.want]
        logits = torch.stack([got[k] for k in order]) if order else None
        if greedy:
            return logits, (self.pick(logits, _GREEDY) if logits is not None else None)
        return logits

    def _sampler(self):
        if getattr(self, "_sampler_obj", None) is None:
            from ..sampling.sampler import Sampler
            self._sampler_obj = Sampler(self.device)
        return self._sampler_obj

    def _context(self, ps: PackedStep, dev: Optional[torch.Tensor] = None) -> StepContext:
        if dev is not None:
            def seg0(name):
                a, m = ps.off[name]
                return dev[a:a + m]
            # a recording: no host-side numbers; max_q is the most rows a sequence can bring (all the step's rows)
            return StepContext(T=ps.T, B=ps.B, tok=seg0("tok"), pos=seg0("pos"), seq=seg0("seq"), slot=seg0("slot"),
                               q_start=seg0("q_start"), kv_len=seg0("kv_len"), h_slot=None, h_q_start=None,
                               h_kv_len=None, decode=ps.decode, max_q=1 if ps.decode else ps.T, max_kv=0,
                               dtype=self.dtype, device=self.device, status=self.status, cache=self.cache,
                               fast=self.dtype == torch.bfloat16, graph=True)
        n = ps.meta.size
        cap = 1 << max(6, (n - 1).bit_length())
        pin = self._pinned.get(cap)
        if pin is None:
            pin = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._pinned[cap] = pin
        # the previous step's copy from this buffer has finished: every step ends in a host read of its results or
        # is followed by another step's copy on the same stream only after this write (copies are stream-ordered
        # and the host waits below before reusing the buffer)
        ev = getattr(self, "_copy_done", None)
        if ev is not None:
            ev.synchronize()
        pin[:n] = torch.from_numpy(ps.meta)
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        dev.copy_(pin[:n], non_blocking=True)
        self._copy_done = torch.cuda.Event()
        self._copy_done.record()
        self._meta_dev = dev

        def seg(name):
            a, m = ps.off[name]
            return dev[a:a + m]
        return StepContext(T=ps.T, B=ps.B, tok=seg("tok"), pos=seg("pos"), seq=seg("seq"), slot=seg("slot"),
                           q_start=seg("q_start"), kv_len=seg("kv_len"), h_slot=ps.h_slot,
                           h_q_start=ps.h_q_start, h_kv_len=ps.h_kv_len, decode=ps.decode, max_q=ps.max_q,
                           max_kv=ps.max_kv, dtype=self.dtype, device=self.device, status=self.status,
                           cache=self.cache, fast=self.dtype == torch.bfloat16)

    def begin_read(self, picked: torch.Tensor):
        """start copying a step's picked tokens and the status word to the host (one pinned buffer, two copies, no
        wait); ``end_read`` of the returned handle waits for them. Two reads may be under way at a time."""
        n = picked.numel()
        ring = getattr(self, "_host_out", None)
        if ring is None or ring[0].numel() < n + 1:
            ring = self._host_out = [torch.empty(max(n + 1, self.max_batch + 1), dtype=torch.int32, pin_memory=True)
                                     for _ in range(2)]
            self._host_turn = 0
        buf = ring[self._host_turn]
        self._host_turn ^= 1
        buf[:n].copy_(picked.view(-1), non_blocking=True)
        buf[n:n + 1].copy_(self.status.view(-1), non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return buf, n, done

    def end_read(self, handle) -> List[int]:
        buf, n, done = handle
        done.synchronize()
        out = buf[:n + 1].tolist()
        if out[n]:
            self._raise_status(out[n])
        return out[:n]

    def read_picked(self, picked: torch.Tensor) -> List[int]:
        """the picked tokens of a step on the host, together with the status check: both are copied into one pinned
        buffer and the host waits for the device once"""
        return self.end_read(self.begin_read(picked))

    def check_status(self) -> None:
        """raise if a kernel of an earlier step met an index it had to skip (waits for the device)"""
        st = int(self.status.item())
        if st:
            self._raise_status(st)

    def _raise_status(self, st: int) -> None:
        if st:
            self.status.zero_()
            from ..kernels import fast
            fast.reset_scratch()
            what = [n for bit, n in ((K.ST_BAD_TOKEN, "a token id outside the vocabulary"),
                                     (K.ST_BAD_PAGE, "a cache position without a mapped page"),
                                     (K.ST_WAIT_TIMEOUT, "a wait inside a kernel ran out"),
                                     (K.ST_BAD_ROW, "a wanted row outside the step")) if st & bit]
            raise EngineError("a kernel reported: %s (status %d); the step's results are not valid"
                              % ("; ".join(what) or "unknown", st))

    # ------------------------------------------------------------------ generation
    def generate_batch(self, prompts, params=None, *, on_tokens=None, cancel=None, **options):
        """generate for a list of prompts (token ids). ``params`` is a ``SamplingParams``; or give its fields as
        keyword options with the reference's names (``temperature``, ``top_p``, ``top_k``, ``min_p``,
        ``repeat_penalty``, ``repeat_last_n``, ``max_tokens``, ``seed``, ``stop_token_ids``). Returns a
        ``GenerationResult`` (``tokens``, ``finish``, ``stats``). The stop tokens are the model's end-of-sequence
        ids plus the given ones."""
        from ..config.runtime import SamplingParams
        from ..sampling.sampler import request_seed
        from .generate import generate
        if params is None:
            params = SamplingParams.from_options(**options)
        elif options:
            params = params.with_(**options)
        stepper = EngineStepper(self, request_seed(params))
        return generate(stepper, prompts, params, stop_token_ids=self.spec.stop_token_ids, on_tokens=on_tokens,
                        cancel=cancel)

    def generate(self, ids, n: int):
        """the greedy continuation of one prompt: exactly ``n`` tokens, stop tokens included, as the reference's
        ``Engine.generate(ids, n)`` (``kindi/nanbeige.py:1317-1325``)"""
        from ..config.runtime import SamplingParams
        from .generate import generate
        stepper = EngineStepper(self, 0)
        return generate(stepper, [list(ids)], SamplingParams(temperature=0.0, max_tokens=n)).tokens[0]

    # ------------------------------------------------------------------ accounting
    def weight_bytes_per_step(self, n_rows: int) -> int:
        return self.model.bytes_read(n_rows)

    def kv_bytes_per_token(self) -> int:
        return self.cache.kv_bytes_per_token()


def _to_run_dtype(t: torch.Tensor, run_dtype: str) -> torch.Tensor:
    from ..weights.loader import target_dtype
    return t.to(target_dtype(t.dtype, run_dtype))


class _StepGraph:
    """the recorded launch sequence of one step shape (a decode step of B sequences, or a prompt step of so many rows,
    sequences and wanted rows), over fixed device buffers"""

    def __init__(self, engine: Engine, ps: PackedStep):
        self.engine = engine
        n = ps.meta.size
        self.pin = torch.empty(n, dtype=torch.int32, pin_memory=True)
        self.pin_np = self.pin.numpy()           # the same memory, written without a tensor operation
        self.meta = torch.zeros(n, dtype=torch.int32, device=engine.device)
        self.meta.copy_(torch.from_numpy(ps.meta))
        self.copied = None
        ctx = engine._context(ps, self.meta)
        a, m = ps.off["rows"]
        rows = self.meta[a:a + m]
        self.graph = torch.cuda.CUDAGraph()
        # Nothing but this library's launches may happen while the stream records: a garbage collection that frees
        # pinned buffers of an earlier engine would query events, which invalidates a recording in the strict mode.
        import gc
        gc.collect()
        torch.cuda.synchronize()
        n0 = K.launch_count()
        was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, capture_error_mode="relaxed"):
                self.logits = engine.model.forward(ctx, rows)
                # the greedy pick rides along (a step that wants no row has nothing to pick)
                self.picked = engine.pick(self.logits, _GREEDY) if self.logits is not None else None
        finally:
            if was_on:
                gc.enable()
        self.launches = K.launch_count() - n0        # recorded, not run
        K.add_launches(-self.launches)

    def replay(self, ps: PackedStep, tokens_from_previous: bool = False) -> torch.Tensor:
        if self.copied is None:
            self.copied = torch.cuda.Event()
        else:
            self.copied.synchronize()            # the pinned buffer is free again
        self.pin_np[:] = ps.meta
        self.meta.copy_(self.pin, non_blocking=True)
        self.copied.record()
        if tokens_from_previous:
            a, n = ps.off["tok"]
            self.meta[a:a + n].copy_(self.engine._picked[:n])      # (before the recording's own pick overwrites them)
        self.graph.replay()
        K.add_launches(self.launches)
        return self.logits


class EngineStepper:
    """what the generation loop drives: the engine's step followed by the sampler, one host read per step; ``launch``
    and ``collect`` split a step so that the next one can be issued while this one runs"""

    def __init__(self, engine: Engine, seed: int):
        self.engine = engine
        self.ctx = engine.ctx
        self.max_positions = engine.spec.max_positions          # the most positions one sequence may reach, or None
        self.max_batch = engine.max_batch
        self.seed = seed
        self._rng: Dict[int, object] = {}

    def alloc(self) -> int:
        return self.engine.alloc()

    def free(self, slot: int) -> None:
        self.engine.free(slot)

    def launch(self, entries, params, seq_ids, histories, tokens_from_previous: bool = False):
        """issue a step and its pick and start reading the picked tokens; returns a handle for ``collect``. With
        ``tokens_from_previous`` the entries' tokens are those the previous step picked, row for row, taken on the
        device: the step can be issued before the previous one has been collected."""
        from ..sampling.sampler import SequenceRandom
        eng = self.engine
        if params.greedy and (params.repeat_penalty == 1.0 or histories is None):
            _, picked = eng.step(entries, greedy=True, tokens_from_previous=tokens_from_previous)
            return eng.begin_read(picked)
        logits = eng.step(entries, tokens_from_previous=tokens_from_previous)
        uniforms = None
        if not params.greedy:
            uniforms = []
            for sid in seq_ids:
                if sid not in self._rng:
                    self._rng[sid] = SequenceRandom(self.seed, sid)
                uniforms.append(self._rng[sid].next())
        picked = eng.pick(logits, params, uniforms, histories if params.repeat_penalty != 1.0 else None)
        return eng.begin_read(picked)

    def collect(self, handle) -> List[int]:
        """the tokens of a launched step (waits for the device)"""
        return self.engine.end_read(handle)

    def run(self, entries, params, seq_ids, histories) -> List[int]:
        return self.collect(self.launch(entries, params, seq_ids, histories))
