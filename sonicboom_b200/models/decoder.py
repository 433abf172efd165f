"""The decoder as a whole: embedding, the blocks in schedule order, final norm, LM head.

One class serves every architecture that can be written as a `ModelSpec`; what differs
between architectures is the spec, not this code.  Order as the reference's emitter walks a
recipe (core/src/model/emit.cpp:237-247 embedding with its optional scale, 436-459 blocks,
512-523 head with its optional logit cap; both are fields of the spec, as the reference keeps
them as traits, core/src/model/recipe.cpp:35-61): the head
runs only on the rows whose logits are wanted (the reference takes the last row only,
core/src/model/gemma4_plan.cpp:599-605), and a tied head reads the embedding matrix
(core/src/model/exec.cpp:516-517).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..parts import BLOCKS, DEPTH_MIXES, NORMS, StepContext, make
from ..weights.loader import TensorRequest


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.blocks = [make(BLOCKS, "block arrangement", l, dtype, device)
                       for l in spec.layers]
        self.final_norm = make(NORMS, "norm", spec.final_norm, dtype, device)
        # per layer: what is handed on instead of the block's own result (None: the result itself)
        self.depth_mixes = [make(DEPTH_MIXES, "depth mix", l.depth_mix, dtype, device)
                            if l.depth_mix is not None else None for l in spec.layers]
        for i, e in enumerate(spec.schedule):
            if e.cache_from is not None:
                mine = self.blocks[e.layer].kv_need()
                theirs = self.blocks[spec.schedule[e.cache_from].layer].kv_need()
                # the mask may differ (the cache then keeps what the widest reader sees), the heads may not
                if mine is None or theirs is None or \
                        (mine.n_kv_heads, mine.head_dim) != (theirs.n_kv_heads, theirs.head_dim):
                    from ..config.specs import ConfigError
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      f"whose keys and values ({theirs}) are not what it needs ({mine})")
        # what joins the stream right before a schedule entry: {entry: StreamInjection}
        self.injections = {inj.before_entry: inj for inj in spec.injections}
        self.injection_vectors = {}
        self.embedding = self.head = self.pair_table = None

    # ------------------------------------------------------------------ weights
    def tensor_requests(self) -> list[TensorRequest]:
        s = self.spec
        req = [TensorRequest(s.embedding_tensor, (s.vocab, s.width), "embedding")]
        for b, m in zip(self.blocks, self.depth_mixes):
            req += b.tensor_requests()
            if m is not None:
                req += m.tensor_requests()
        req += self.final_norm.tensor_requests()
        if s.pair_embedding is not None:
            req.append(TensorRequest(s.pair_embedding.tensor, (s.pair_embedding.buckets + 1, s.width), "embedding"))
        req += [TensorRequest(inj.tensor, (inj.rows, s.width), "bias") for inj in s.injections if inj.tensor]
        req += [TensorRequest(name, tuple(shape), optional=True) for name, shape in s.unused_tensors]
        if s.head_tensor is not None:
            req.append(TensorRequest(s.head_tensor, (s.vocab, s.width)))
        else:
            # a tied model's file may still carry a copy of the head; it is not read
            req.append(TensorRequest("lm_head.weight", (s.vocab, s.width), optional=True))
        return req

    def bind(self, get) -> None:
        self.embedding = get(self.spec.embedding_tensor)
        if self.spec.pair_embedding is not None:
            self.pair_table = get(self.spec.pair_embedding.tensor)
            if self.pair_table.dtype != self.embedding.dtype:
                self.pair_table, self.embedding = self.pair_table.float(), self.embedding.float()
        for b, m in zip(self.blocks, self.depth_mixes):
            b.bind(get)
            if m is not None:
                m.bind(get)
        self.final_norm.bind(get)
        tables = {}
        for e, inj in self.injections.items():
            if inj.tensor:
                if inj.tensor not in tables:
                    tables[inj.tensor] = get(inj.tensor)
                self.injection_vectors[e] = tables[inj.tensor][inj.row]
        self.head = self.embedding if self.spec.head_tensor is None else get(self.spec.head_tensor)

    # ------------------------------------------------------------------ what the cache must hold
    def kv_needs(self) -> list:
        """Per schedule entry: its KVNeed, or None when it reads another entry's cache.  An entry
        whose cache others read keeps what the reader with the widest mask sees."""
        from ..cache.kv import KVNeed
        needs = [self.blocks[e.layer].kv_need() if e.cache_from is None else None
                 for e in self.spec.schedule]
        for e in self.spec.schedule:
            if e.cache_from is None:
                continue
            mine, own = self.blocks[e.layer].kv_need(), needs[e.cache_from]
            window = 0 if 0 in (mine.window, own.window) else max(mine.window, own.window)
            needs[e.cache_from] = KVNeed(own.n_kv_heads, own.head_dim, window,
                                         max(mine.keep_first, own.keep_first) if window else 0)
        return needs

    def state_needs(self) -> list:
        return [self.blocks[e.layer].state_need() for e in self.spec.schedule]

    def model_state_needs(self) -> dict:
        """Named per-sequence state that belongs to no schedule entry: the last token a sequence was
        fed, which a pair embedding hashes with the next one."""
        from ..cache.kv import StateNeed
        return {"prev_token": StateNeed((), torch.int32)} if self.spec.pair_embedding is not None else {}

    # ------------------------------------------------------------------ one step
    def forward(self, plan, cache) -> torch.Tensor:
        """Runs the step's rows through every schedule entry; returns float32 logits
        [len(plan.want_rows), vocab] (None when no logits are wanted)."""
        s = self.spec
        n = len(s.schedule)
        mixes = [self.depth_mixes[e.layer] for e in s.schedule]
        # With depth mixing the embedding output and every block result of the step are kept side
        # by side: streams[0] is the embedding output, streams[i + 1] the result of entry i.
        streams = torch.empty((n + 1, plan.n_rows, s.width), dtype=torch.float32, device=self.device) \
            if any(m is not None for m in mixes) else None
        x = streams[0] if streams is not None else \
            torch.empty((plan.n_rows, s.width), dtype=torch.float32, device=self.device)
        ctx = StepContext(plan=plan, cache=cache)
        if s.pair_embedding is None:
            ops.embed(plan.tokens, self.embedding, x, s.embedding_scale)
        else:
            pe, prev = s.pair_embedding, ctx.model_state("prev_token")
            ops.embed_pair(plan, prev, self.embedding, self.pair_table, pe.buckets, pe.mul_prev, pe.mul_cur, x,
                           s.embedding_scale)
            ops.keep_last_token(plan, prev)
        # an injection may add the embedding output again: it is then kept apart from the stream,
        # which blocks overwrite
        embedded = x if any(inj.embedding for inj in self.injections.values()) else None
        for i, e in enumerate(s.schedule):
            if i in self.injections or x is embedded:
                x = self._inject(self.injections.get(i), i, x, embedded, self.blocks[e.layer], ctx)
            ctx.entry = i
            ctx.owns_cache = e.cache_from is None
            ctx.kv_entry = i if e.cache_from is None else e.cache_from
            block, mix = self.blocks[e.layer], mixes[i]
            # the next entry's first norm can ride on this entry's last product
            nxt = self.blocks[s.schedule[i + 1].layer] if i + 1 < n else None
            next_norm = nxt.input_norm() if nxt is not None else None
            if i + 1 in self.injections:
                next_norm = nxt = None          # the stream changes before the next entry reads it
            ctx.after_block_norm = next_norm if mix is None else None
            # ... and its first weights can be asked into L2 meanwhile, if it would ask late
            ctx.after_block_weights = nxt.first_weights(plan.n_rows) if nxt is not None and mix is None else None
            if streams is not None:
                if getattr(block, "writes_block_out", False):
                    ctx.block_out = streams[i + 1]
                    # the block may run the mix together with its last residual add
                    ctx.block_mix = (mix, streams, next_norm) if mix is not None and hasattr(mix, "joins") else None
                elif x.data_ptr() == streams[i].data_ptr():
                    x = ops.depth_mix(streams[i:i + 1], 1, self._one(), torch.empty_like(x))   # the block may overwrite its input
            with ops.trace_range(f"entry {i} (layer {e.layer})"):
                x = block.forward(x, ctx)
            ctx.block_out = ctx.block_mix = None
            mixed, ctx.mixed_out = ctx.mixed_out, None
            if streams is None:
                continue
            if mixed is not None:
                x = mixed
                continue
            if x.data_ptr() != streams[i + 1].data_ptr():
                ops.depth_mix(x.unsqueeze(0), 1, self._one(), streams[i + 1])
                x = streams[i + 1]
            if mix is not None:
                x = self._mix(mix, streams, ctx, next_norm)
        if plan.n_want == 0:
            return None
        hn = self.final_norm.forward(x, self.dtype, rows=plan.want_rows)
        logits = torch.empty((plan.n_want, s.vocab), dtype=torch.float32, device=self.device)
        ops.linear(hn, self.head, logits)
        if s.logit_scale != 1.0:
            ops.scale(logits, s.logit_scale)
        return ops.softcap(logits, s.logit_cap) if s.logit_cap > 0.0 else logits


    def _inject(self, inj, entry, x, embedded, block, ctx):
        """x + the embedding output (if asked) + the injection's vector, with the block's first norm
        written along; without an injection, a copy of the embedding output that the block may
        overwrite."""
        out = x if x is not embedded else torch.empty_like(x)
        norm = block.input_norm()
        rms = norm.as_rms() if norm is not None else None
        ride = None
        if rms is not None:
            ride = (rms[0], rms[1], torch.empty(x.shape, dtype=self.dtype, device=self.device))
        ops.stream_add(x, embedded if inj is not None and inj.embedding else None,
                       self.injection_vectors.get(entry) if inj is not None else None, out, ride)
        if ride is not None:
            ctx.keep_normed(norm, out, ride[2])
        return out

    def _one(self):
        if getattr(self, "_one_coef", None) is None:
            self._one_coef = torch.ones(1, dtype=torch.float32, device=self.device)
        return self._one_coef

    def _mix(self, mix, streams, ctx, next_norm):
        """What a depth mix hands on; the next entry's first norm is written with it when that
        is a plain RMS norm."""
        out = torch.empty(streams.shape[1:], dtype=torch.float32, device=self.device)
        rms = next_norm.as_rms() if next_norm is not None else None
        if rms is None:
            return mix.forward(streams, out)
        normed = torch.empty(out.shape, dtype=self.dtype, device=self.device)
        mix.forward(streams, out, (rms[0], rms[1], normed))
        ctx.keep_normed(next_norm, out, normed)
        return out


def tensor_requests(spec: ModelSpec) -> list[TensorRequest]:
    """Tensors a model of this spec wants; no device is touched."""
    return DecoderModel(spec, torch.float32, "cpu").tensor_requests()
