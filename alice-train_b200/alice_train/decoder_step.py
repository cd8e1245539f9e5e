"""The ternary linears of a whole decoder as one data-parallel QAT micro-step.

The reference's trainers walk the layers and, per projection, quantise the latent weights and run the forward, dx
and dW products (src/bin/train_qat_70b.rs:885-917,1157-1229 for Llama; src/bin/train_qat_qwen35.rs:839,922 with
Qwen35LayerWeights::fake_quantize, src/qwen35.rs:366-437).  Here the same sequence for every linear of the model is
handed to the library in ONE call (ab_qat_linear_steps), tokens split over the GPUs, dW of every linear summed over
the GPUs inside NVSwitch while the following kernels run.  Attention, DeltaNet state updates, norms and the lm_head
are not ternary linears and are not part of this step; every linear gets its own synthetic x and dy of the right shape.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _ffi
from .bitlinear import BitLinearWeights


def llama_linears(hidden: int, intermediate: int, heads: int, kv_heads: int, head_dim: int):
    """(name, out_features, in_features) of one Llama decoder layer: q, k, v, o, gate, up, down
    (src/llama.rs:183-203; LlamaConfig::llama3_1b src/llama.rs:64-80, llama3_70b :100-116)."""
    q, kv = heads * head_dim, kv_heads * head_dim
    return [("q_proj", q, hidden), ("k_proj", kv, hidden), ("v_proj", kv, hidden), ("o_proj", hidden, q),
            ("gate_proj", intermediate, hidden), ("up_proj", intermediate, hidden), ("down_proj", hidden, intermediate)]


def qwen35_layer_linears(full_attention: bool, hidden: int = 4096, intermediate: int = 12288):
    """Qwen3.5-9B (Qwen35Config::qwen35_9b, src/qwen35.rs:70-102): a Gated-DeltaNet layer has in_proj_qkv, in_proj_z,
    in_proj_b, in_proj_a, out_proj (src/qwen35.rs:154-164), a full-attention layer q, k, v, o (:183-191); both carry
    the gate / up / down MLP."""
    mlp = [("gate_proj", intermediate, hidden), ("up_proj", intermediate, hidden), ("down_proj", hidden, intermediate)]
    if full_attention:
        attn, kv = 16 * 256, 4 * 256
        return [("q_proj", attn, hidden), ("k_proj", kv, hidden), ("v_proj", kv, hidden), ("o_proj", hidden, attn)] + mlp
    key, val, v_heads = 16 * 128, 32 * 128, 32
    return [("in_proj_qkv", 2 * key + val, hidden), ("in_proj_z", val, hidden), ("in_proj_b", v_heads, hidden),
            ("in_proj_a", v_heads, hidden), ("out_proj", hidden, val)] + mlp


MODELS = {
    # name: (tokens per step, list of layers, each a list of linears, std of the latent weights, gamma guard)
    "llama32-1b-qat": lambda: (8192, [llama_linears(2048, 8192, 32, 8, 64) for _ in range(16)], 0.02, _ffi.AB_GUARD_FLOOR),
    "qwen35-9b-hybrid": lambda: (8192, [qwen35_layer_linears((i + 1) % 4 == 0) for i in range(32)], 0.02, _ffi.AB_GUARD_INV_ZERO),
    "llama-tiny": lambda: (512, [llama_linears(256, 512, 4, 2, 64) for _ in range(2)], 0.02, _ffi.AB_GUARD_FLOOR),
}


class DataParallelQatStep:
    """Latent weights, weight handles, gradient buffers and work buffers of every linear of a model, and the call that
    runs one micro-step over all of them.  `tokens` are THIS GPU's tokens.  exchange: "switch" (dW in symmetric memory,
    summed inside NVSwitch by the library), "nccl" (torch.distributed all-reduce per linear) or "none"."""

    def __init__(self, ctx, layers, tokens: int, device, weight_std: float = 0.02, guard: int = _ffi.AB_GUARD_FLOOR,
                 exchange: str = "none", ctas: int = 0, seed: int = 0, quantise_in_step: bool = True):
        self.ctx, self.tokens, self.device, self.guard, self.ctas = ctx, int(tokens), device, guard, int(ctas)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.exchange = exchange if self.world > 1 else "none"
        self.quantise_in_step = quantise_in_step
        self.linears = [(li, name, out, inn) for li, layer in enumerate(layers) for (name, out, inn) in layer]
        self.params = sum(o * i for _, _, o, i in self.linears)
        gen = torch.Generator(device=device)
        m = self.tokens
        # activations and outputs: one buffer per distinct shape, shared by the linears of that shape (stream order
        # keeps the uses apart); every rank draws its own tokens
        self._act, self._grad, self._y, self._dx = {}, {}, {}, {}
        for _, _, out, inn in self.linears:
            if inn not in self._act:
                gen.manual_seed(1000 + 97 * self.rank + inn)
                self._act[inn] = torch.randn((m, inn), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
                self._dx[inn] = torch.empty((m, inn), dtype=torch.bfloat16, device=device)
            if out not in self._grad:
                gen.manual_seed(2000 + 97 * self.rank + out)
                self._grad[out] = (torch.randn((m, out), generator=gen, device=device, dtype=torch.float32) * 1e-2).to(torch.bfloat16)
                self._y[out] = torch.empty((m, out), dtype=torch.bfloat16, device=device)
        kmax = max(i for _, _, _, i in self.linears)
        self._xq = torch.empty((m, kmax), dtype=torch.int8, device=device)
        self._scales = torch.empty(m, dtype=torch.float32, device=device)
        self._rowsums = torch.empty(m, dtype=torch.int32, device=device)
        # latent weights (identical on every rank: data parallel) and handles
        self.latent, self.weights = [], []
        for idx, (li, name, out, inn) in enumerate(self.linears):
            gen.manual_seed(seed + 10 + idx)
            w_lat = torch.randn((out, inn), generator=gen, device=device, dtype=torch.float32) * weight_std
            self.latent.append(w_lat)
            self.weights.append(BitLinearWeights(out, inn, ctx).quantize_(w_lat, guard=guard))
        # gradient buffers: one symmetric-memory arena per layer when the switch sums them
        self.arenas, self.dW, self._xchg = [], [None] * len(self.linears), [None] * len(self.linears)
        if self.exchange == "switch":
            from .parallel import SwitchArena
            by_layer = {}
            for idx, (li, *_rest) in enumerate(self.linears):
                by_layer.setdefault(li, []).append(idx)
            for li in sorted(by_layer):
                ids = by_layer[li]
                arena = SwitchArena(ctx, [4 * self.linears[i][2] * self.linears[i][3] for i in ids], device)
                self.arenas.append(arena)
                for slot, i in enumerate(ids):
                    _, _, out, inn = self.linears[i]
                    self.dW[i] = arena.view(slot, torch.float32, (out, inn))
                    self._xchg[i] = arena.pointers(slot)
            torch.cuda.synchronize(device)
            dist.barrier()
            torch.cuda.synchronize(device)
        else:
            for i, (_, _, out, inn) in enumerate(self.linears):
                self.dW[i] = torch.zeros((out, inn), dtype=torch.float32, device=device)
        self._epoch = 0
        self._steps = (_ffi.LinearStep * len(self.linears))()
        for i, (_, _, out, inn) in enumerate(self.linears):
            s = self._steps[i]
            s.w = self.weights[i].handle.value
            s.w_latent = self.latent[i].data_ptr() if quantise_in_step else None
            s.x_bf16, s.dy_bf16 = self._act[inn].data_ptr(), self._grad[out].data_ptr()
            s.xq, s.scales, s.rowsums = self._xq.data_ptr(), self._scales.data_ptr(), self._rowsums.data_ptr()
            s.y_bf16, s.dx_bf16 = self._y[out].data_ptr(), self._dx[inn].data_ptr()
            s.dW, s.dw_beta = self.dW[i].data_ptr(), 0.0
            if self._xchg[i] is not None:
                _, mc, fl, fmc = self._xchg[i]
                s.dw_multicast, s.flags_local, s.flags_multicast = mc, fl, fmc
        ctx.sync()

    # ------------------------------------------------------------------------------------------------
    def step(self):
        """One micro-step over every linear (asynchronous on the context's stream)."""
        lib = _ffi.load()
        if self.exchange == "nccl":
            pending = []
            for i in range(len(self.linears)):
                _ffi.check(lib.ab_qat_linear_steps(self.ctx.handle, C.byref(self._steps[i]), 1, self.tokens, self.guard,
                                                   self.rank, self.world, 1, self.ctas), self.ctx.handle)
                pending.append(dist.all_reduce(self.dW[i], op=dist.ReduceOp.SUM, async_op=True))
            for h in pending:
                h.wait()
            return
        self._epoch += 1
        _ffi.check(lib.ab_qat_linear_steps(self.ctx.handle, self._steps, len(self.linears), self.tokens, self.guard,
                                           self.rank, self.world, self._epoch, self.ctas), self.ctx.handle)

    # ------------------------------------------------------------------------------------------------
    def check_exchange(self, max_linears: int = 0):
        """Correctness evidence for the in-switch sum, run between steps (collective).  For each checked buffer:
        (a) a rank-dependent pattern of small integers is summed by the switch and compared, bit for bit, with the
        sum every rank can compute on its own (integer sums are exact in any order); (b) the dW of a real micro-step
        is summed by the switch and, from a copy, by NCCL: bit-identical at 2 GPUs, otherwise within a few units in the
        last place of the largest element (the two reductions add in different orders).  Returns a dict; raises
        RuntimeError on a mismatch."""
        if self.exchange != "switch":
            return {"checked": 0, "note": "no in-switch exchange in this run"}
        lib = _ffi.load()
        ids = list(range(len(self.linears)))
        if max_linears and len(ids) > max_linears:      # spread over the model: first, last and evenly between
            stride = max(1, len(ids) // max_linears)
            ids = sorted(set(ids[::stride][:max_linears - 1] + [ids[-1]]))
        worst, identical, total = 0.0, 0, 0
        for i in ids:
            _, name, out, inn = self.linears[i]
            buf = self.dW[i]
            n = buf.numel()
            _, mc, fl, fmc = self._xchg[i]
            idx = torch.arange(n, device=self.device, dtype=torch.int64)
            # (a) integer pattern
            expect = torch.zeros(n, device=self.device, dtype=torch.float32)
            for r in range(self.world):
                expect += (((idx * 7 + r * 13) % 251) - 125).to(torch.float32)
            buf.view(-1).copy_((((idx * 7 + self.rank * 13) % 251) - 125).to(torch.float32))
            self._exchange_one(lib, mc, n, fl, fmc, i)
            if not torch.equal(buf.view(-1), expect):
                bad = int((buf.view(-1) != expect).sum().item())
                raise RuntimeError(f"in-switch all-reduce of {name} [{out}x{inn}]: {bad} of {n} integer sums differ")
            # (b) real gradient against NCCL
            st = self._steps[i]
            keep = (st.dw_multicast, st.w_latent)
            st.dw_multicast, st.w_latent = None, None
            _ffi.check(lib.ab_qat_linear_steps(self.ctx.handle, C.byref(st), 1, self.tokens, self.guard, self.rank,
                                               self.world, 1, self.ctas), self.ctx.handle)
            st.dw_multicast, st.w_latent = keep
            ref = buf.clone()
            dist.all_reduce(ref, op=dist.ReduceOp.SUM)
            self._exchange_one(lib, mc, n, fl, fmc, i)
            diff = (buf - ref).abs().max().item()
            scale = ref.abs().max().item()
            total += 1
            if torch.equal(buf, ref):
                identical += 1
            rel = diff / scale if scale > 0 else 0.0
            worst = max(worst, rel)
            if rel > 1e-6 or (self.world == 2 and diff != 0.0):
                raise RuntimeError(f"in-switch all-reduce of {name} [{out}x{inn}] differs from NCCL: max |diff| {diff:.3e} "
                                   f"of {scale:.3e}")
            del ref, expect, idx
        return {"checked": total, "integer_pattern": "bit-exact", "vs_nccl_bit_identical": identical,
                "vs_nccl_max_rel_diff": worst}

    def _exchange_one(self, lib, mc, n, fl, fmc, i):
        # the counters of buffer i advance with every exchange on it: all buffers share the step's epoch, so a check
        # exchanges every buffer's epoch past the step count; keep them in step by using (and bumping) a per-buffer epoch
        ep = self._buf_epoch(i)
        _ffi.check(lib.ab_dp_allreduce_start(self.ctx.handle, mc, n, fl, fmc, self.rank, self.world, ep, self.ctas), self.ctx.handle)
        _ffi.check(lib.ab_dp_allreduce_wait(self.ctx.handle), self.ctx.handle)
        self.ctx.sync()

    def _buf_epoch(self, i):
        if not hasattr(self, "_check_epochs"):
            self._check_epochs = {}
        e = self._check_epochs.get(i, self._epoch) + 1
        self._check_epochs[i] = e
        return e

    def resync_epochs(self):
        """After check_exchange the buffers' counters differ (checked buffers ran extra exchanges): zero all counters
        collectively and restart the epoch count so that step() is consistent again."""
        for a in self.arenas:
            a.reset_flags()
        self._epoch = 0
        self._check_epochs = {}

    def close(self):
        for w in self.weights:
            w.close()
        self.weights, self.latent, self.dW, self.arenas = [], [], [], []
