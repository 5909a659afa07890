"""GPT-2 pipeline stage on the sm_100a kernels.

No autograd and no nn.Module: the stage owns five flat buffers (fp32 master
weights, fp32 main gradient, Adam moments, bf16 compute copy of the weights)
and runs an explicit forward and backward through the kernels in ops/.  The
flat layout is what lets the optimiser be one kernel and the two stage-wide
synchronisations be single fused kernels over peer memory (the weights and the
gradient live in symmetric buffers that the other replicas of the stage map).

Numerics: bf16 activations and GEMM operands with fp32 accumulation, fp32
LayerNorm statistics / softmax / loss, fp32 master weights, gradients and
optimiser state.  The reference trains with bf16 autocast over fp32 parameters
(src/train.py:199, src/config.py:37-40); its residual stream stays fp32, here
it is bf16.

Reference: ShardedGPT2.forward / backward (src/model.py:200-209) and the
optimiser / DiLoCo part of train_step (src/train.py:247-269).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .gpt2 import GPT2Config, init_tensor, split_layers, stage_param_specs
from ..ops import kernels as K
from ..ops._lib import Status, load_all_kernels
from ..ops.attention import attention_bwd, attention_fwd
from ..parallel.collectives import GradSync, OuterSync, StageRendezvous, wait_cycles_for
from ..parallel.symm import SymmetricBuffer

BF16, F32 = torch.bfloat16, torch.float32


def _align(n: int, a: int = 8) -> int:
    return (n + a - 1) // a * a


class _BlockView:
    """Parameter views (fp32 master, bf16 copy, fp32 gradient) of one block."""
    pass


class B200Engine:
    name = "b200"

    def __init__(self, cfg: GPT2Config, world, config, device: torch.device):
        assert device.type == "cuda", "the b200 engine needs a CUDA device"
        self.cfg, self.world, self.config, self.device = cfg, world, config, device
        S = world.num_stages
        self.is_first, self.is_last = world.stage == 0, world.stage == S - 1
        self.layers = split_layers(cfg.n_layer, S, config.swarm.layer_split, cfg.n_embd, cfg.vocab_size)[world.stage]
        self.specs = stage_param_specs(cfg, self.layers, self.is_first, self.is_last)
        self.act_dtype = BF16
        self.status = Status(device)
        d = cfg.n_embd
        assert d % 8 == 0 and cfg.vocab_size % 8 == 0, "n_embd and vocab_size must be multiples of 8"
        assert cfg.bias, "the b200 engine implements the reference's bias=True model"
        if cfg.dropout != 0.0:
            raise NotImplementedError(
                "model.dropout > 0 is implemented by the autograd engine only (--engine torch); the sm_100a "
                "kernels train without dropout, as every configuration and experiment of the reference does")
        K.set_deterministic(bool(getattr(config.train, "deterministic", False)))
        self.head_chunks = max(1, int(getattr(config.train, "lm_head_chunks", 1)))

        # ---- flat layout ------------------------------------------------
        self.offsets: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        off = 0
        for key, _, shape in self.specs:
            self.offsets[key] = (off, shape)
            off += _align(math.prod(shape))
        self.n = _align(off, 8 * 8)          # divisible into 8-element-aligned shards for up to 8 replicas
        group = world.curr_stage_group if world.num_replicas > 1 else None
        nvls = config.swarm.collective == "nvls"
        self.theta_buf = SymmetricBuffer(self.n * 4, device, group, multicast=nvls)
        self.grad_buf = SymmetricBuffer(self.n * 4, device, group, multicast=nvls)
        self.theta = self.theta_buf.view(F32, self.n)
        self.grad = self.grad_buf.view(F32, self.n)
        self.w16 = torch.zeros(self.n, dtype=BF16, device=device)
        self.m = torch.zeros(self.n, dtype=F32, device=device)
        self.v = torch.zeros(self.n, dtype=F32, device=device)
        self.stats = torch.zeros(4, dtype=F32, device=device)        # sumsq, norm, clip coef
        self.count_buf = torch.zeros(1, dtype=F32, device=device)
        for key, gname, shape in self.specs:
            self.p32(key).copy_(init_tensor(gname, shape, config.train.seed, cfg.n_layer))
        K.cast_to_bf16(self.theta, self.w16)

        ic = config.train.inner_optimizer
        self.inner_type = ic.type
        self.inner_cfg = ic
        self.mom_inner = torch.zeros(self.n, dtype=F32, device=device) if ic.type == "SGD" and ic.momentum else None
        self.opt_step = 0
        oc = config.train.outer_optimizer
        self.has_outer = oc.type != "None"
        self.fused = config.swarm.collective in ("fused", "nvls")
        self.outer: Optional[OuterSync] = None
        if self.has_outer:
            assert oc.type == "SGD", "the outer optimiser is SGD (optionally Nesterov) as in the reference"
            self.outer = OuterSync(self.theta_buf, self.n, device, oc.lr, oc.momentum, oc.nesterov, group, self.status,
                                   wait_cycles=wait_cycles_for(config.swarm.peer_wait_s))
        self.grad_sync = GradSync(self.grad_buf, self.n, device, group,
                                  wire_bf16=config.swarm.grad_wire_dtype == "bfloat16", status=self.status,
                                  wait_cycles=wait_cycles_for(config.swarm.peer_wait_s))
        self.rendezvous = StageRendezvous(group, device)
        self.stash: Dict[int, dict] = {}
        self.training = True
        self._build_views()
        load_all_kernels()
        # Weight-gradient GEMMs and bias column sums are off the backward critical path (nothing in the
        # backward reads them), so they run on a second stream and fill the SMs that the dgrad chain,
        # LayerNorm and attention kernels leave idle (last partial waves, memory-bound phases).
        self.side = torch.cuda.Stream(device) if os.environ.get("DSWARM_WGRAD_STREAM", "1") != "0" else None
        self._side_dirty = False
        # Gradient buckets in the order the backward pass completes them (head, blocks from last to
        # first, embeddings).  During the last backward of a step that ends with a gradient sync, each
        # bucket's fused all-reduce is queued on its own stream as soon as the bucket is final, so the
        # NVLink traffic runs under the rest of the backward pass.
        self.comm_stream = torch.cuda.Stream(device)
        self.buckets = self._make_buckets()
        self._buckets_sent = 0
        self._overlap = os.environ.get("DSWARM_GRAD_OVERLAP", "1") != "0"
        self._canary_every_step = os.environ.get("DSWARM_CANARY_CHECK", "0") == "1"

    # ------------------------------------------------------------------ views
    def _slice(self, buf: torch.Tensor, key: str) -> torch.Tensor:
        off, shape = self.offsets[key]
        return buf[off:off + math.prod(shape)].view(shape)

    def p32(self, key: str) -> torch.Tensor:
        return self._slice(self.theta, key)

    def p16(self, key: str) -> torch.Tensor:
        return self._slice(self.w16, key)

    def g32(self, key: str) -> torch.Tensor:
        return self._slice(self.grad, key)

    def _build_views(self) -> None:
        self.blocks: List[_BlockView] = []
        for li in range(len(self.layers)):
            b = _BlockView()
            pre = f"transformer.h.{li}."
            for short, name in (("ln1", "ln_1"), ("ln2", "ln_2")):
                setattr(b, f"{short}_w", self.p32(pre + name + ".weight"))
                setattr(b, f"{short}_b", self.p32(pre + name + ".bias"))
                setattr(b, f"d{short}_w", self.g32(pre + name + ".weight"))
                setattr(b, f"d{short}_b", self.g32(pre + name + ".bias"))
            for short, name in (("qkv", "attn.c_attn"), ("o", "attn.c_proj"), ("fc", "mlp.c_fc"), ("pr", "mlp.c_proj")):
                setattr(b, f"{short}_w", self.p16(pre + name + ".weight"))
                setattr(b, f"{short}_b", self.p32(pre + name + ".bias"))
                setattr(b, f"d{short}_w", self.g32(pre + name + ".weight"))
                setattr(b, f"d{short}_b", self.g32(pre + name + ".bias"))
            self.blocks.append(b)
        if self.is_first:
            self.wte, self.wpe = self.p32("transformer.wte.weight"), self.p32("transformer.wpe.weight")
            self.dwte, self.dwpe = self.g32("transformer.wte.weight"), self.g32("transformer.wpe.weight")
        if self.is_last:
            self.lnf_w, self.lnf_b = self.p32("transformer.ln_f.weight"), self.p32("transformer.ln_f.bias")
            self.dlnf_w, self.dlnf_b = self.g32("transformer.ln_f.weight"), self.g32("transformer.ln_f.bias")
            hk = "lm_head.weight" if "lm_head.weight" in self.offsets else "transformer.wte.weight"
            self.head_w, self.dhead_w = self.p16(hk), self.g32(hk)

    # ------------------------------------------------------------------ small API
    def train(self):
        self.training = True

    def eval(self):
        self.training = False

    def zero_grad(self) -> None:
        if self.opt_step == 0:
            self.grad.zero_()        # afterwards the optimiser kernel clears it

    def num_parameters(self) -> int:
        n = sum(math.prod(s) for _, _, s in self.specs)
        if self.is_first:
            n -= self.cfg.block_size * self.cfg.n_embd
        return n

    def check_status(self) -> None:
        self.status.raise_if_set()
        if self._canary_every_step:
            for buf in self.symmetric_buffers():
                buf.check_canaries()

    def symmetric_buffers(self):
        """Every peer-mapped buffer of this stage (weights, gradient, the collectives' flags and staging)."""
        out = [self.theta_buf, self.grad_buf]
        for obj in (self.outer, self.grad_sync):
            for name in ("flags", "stage_buf"):
                b = getattr(obj, name, None) if obj is not None else None
                if b is not None:
                    out.append(b)
        return out

    def warmup(self, B: int, T: int) -> None:
        """Run every code path of a step once on dummy data of the real shape, then
        put the state back.  Library kernels (attention, copies) are loaded on first
        use, and a first use that happens while a pipeline receive is spinning on the
        device can wait forever; after this pass nothing is loaded inside a step."""
        dev, d = self.device, self.cfg.n_embd
        theta0 = self.theta.clone()
        ids = torch.zeros(B, T, dtype=torch.long, device=dev) if self.is_first else None
        hidden = torch.zeros(B, T, d, dtype=BF16, device=dev) if not self.is_first else None
        tg = torch.zeros(B, T, dtype=torch.long, device=dev)
        mask = torch.ones(B, T, dtype=torch.long, device=dev)
        if self.is_last:
            self.forward_backward(-1, ids, hidden, tg, mask, 1.0)
            self.forward_loss(ids, hidden, tg, mask, 1.0)
        else:
            y = self.forward(-1, ids, hidden)
            self.backward(-1, torch.zeros_like(y))
            self.forward(-1, ids, hidden, keep=False)
        self.forward_infer(ids, hidden)
        self.optimizer_step(0.0, 1.0)
        torch.cuda.synchronize(dev)
        self.theta.copy_(theta0)
        K.cast_to_bf16(self.theta, self.w16)
        for t in (self.grad, self.m, self.v, self.stats):
            t.zero_()
        if self.mom_inner is not None:
            self.mom_inner.zero_()
        self.opt_step = 0
        self.status.word.zero_()
        self.stash.clear()
        torch.cuda.synchronize(dev)

    def _make_buckets(self) -> List[Tuple[int, int]]:
        groups: List[List[str]] = []
        if self.is_last:
            groups.append([k for k, _, _ in self.specs if k.startswith("transformer.ln_f") or k.startswith("lm_head")])
        for li in reversed(range(len(self.layers))):
            groups.append([k for k, _, _ in self.specs if k.startswith(f"transformer.h.{li}.")])
        if self.is_first:
            groups.append([k for k, _, _ in self.specs if k.startswith("transformer.wte") or k.startswith("transformer.wpe")])
        ends = sorted(off for off, _ in self.offsets.values()) + [self.n]
        out = []
        for g in groups:
            if not g:
                continue
            lo = min(self.offsets[k][0] for k in g)
            hi = max(self.offsets[k][0] for k in g)
            hi = min(e for e in ends if e > hi)          # start of the next tensor (offsets are 8-aligned)
            out.append((lo, hi - lo))
        covered = sum(c for _, c in out)
        assert covered == self.n, (covered, self.n)
        return out

    def _send_bucket(self) -> None:
        """Queue the next bucket's all-reduce behind everything queued so far on the compute streams."""
        off, cnt = self.buckets[self._buckets_sent]
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        if self.side is not None:
            self.comm_stream.wait_stream(self.side)
        if self._buckets_sent == 0:
            # replicas reach their last backward at different times (routing gives them different loads):
            # meet on the communication stream first, so the kernels' bounded peer waits only see the
            # microseconds between the replicas leaving that meeting, not the skew of the step
            self.rendezvous.meet(self.comm_stream)
        self.grad_sync.bucket(off, cnt, stream=self.comm_stream)
        self._buckets_sent += 1

    def _fork(self, *tensors):
        """Context for work that may run beside the main stream: waits for what has been queued on
        the main stream so far and pins the given tensors' memory until the side work is done."""
        eng = self

        class _Ctx:
            def __enter__(self_inner):
                if eng.side is None:
                    return None
                eng.side.wait_stream(torch.cuda.current_stream())
                for t in tensors:
                    t.record_stream(eng.side)
                self_inner.cm = torch.cuda.stream(eng.side)
                self_inner.cm.__enter__()
                eng._side_dirty = True
                return eng.side

            def __exit__(self_inner, *exc):
                if eng.side is not None:
                    self_inner.cm.__exit__(*exc)
                return False
        return _Ctx()

    def _join(self) -> None:
        """Main stream waits for the side stream (before anything reads the gradients)."""
        if self.side is not None and self._side_dirty:
            torch.cuda.current_stream().wait_stream(self.side)
            self._side_dirty = False

    # ------------------------------------------------------------------ forward pieces
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        return K.embedding_fwd(ids.contiguous(), self.wte, self.wpe, self.status)

    def _block_fwd(self, b: _BlockView, x: torch.Tensor, B: int, T: int, keep: bool):
        st = self.status
        ln1, mu1, rs1 = K.layernorm_fwd(x, b.ln1_w, b.ln1_b)
        qkv = K.gemm(ln1, b.qkv_w, bias=b.qkv_b, status=st)
        att, actx = attention_fwd(qkv, B, T, self.cfg.n_head, need_ctx=keep, status=st)
        x1 = K.gemm(att, b.o_w, mode=K.EPI_RESID, bias=b.o_b, resid=x, status=st)
        ln2, mu2, rs2 = K.layernorm_fwd(x1, b.ln2_w, b.ln2_b)
        # the GELU epilogue also emits gelu'(pre-activation): the backward then only multiplies
        h = torch.empty(x.shape[0], 4 * x.shape[1], dtype=BF16, device=x.device) if keep else None
        g = K.gemm(ln2, b.fc_w, mode=K.EPI_GELU, bias=b.fc_b, aux_out=h, status=st)
        x2 = K.gemm(g, b.pr_w, mode=K.EPI_RESID, bias=b.pr_b, resid=x1, status=st)
        saved = (x, ln1, mu1, rs1, actx, att, x1, ln2, mu2, rs2, h, g) if keep else None
        return x2, saved

    def _block_bwd(self, b: _BlockView, saved, dx2: torch.Tensor) -> torch.Tensor:
        st = self.status
        x, ln1, mu1, rs1, actx, att, x1, ln2, mu2, rs2, h, g = saved
        Mtok = x.shape[0]
        d = x.shape[1]
        dh = K.gemm(dx2, b.pr_w, b_t=False, mode=K.EPI_MUL, aux_in=h, status=st)
        with self._fork(dx2, g, dh, ln2):
            K.gemm(dx2, g, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=b.dpr_w,
                   split_k=K.wgrad_split(d, 4 * d, Mtok), status=st)
            K.colsum_accum(dh, b.dfc_b)
            K.gemm(dh, ln2, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=b.dfc_w,
                   split_k=K.wgrad_split(4 * d, d, Mtok), status=st)
        dln2 = K.gemm(dh, b.fc_w, b_t=False, status=st)
        # the column sum of dx2 (bias gradient of mlp.c_proj) rides along with the LayerNorm backward
        dx1 = K.layernorm_bwd(dln2, x1, b.ln2_w, mu2, rs2, b.dln2_w, b.dln2_b, dres=dx2, dres_sum=b.dpr_b)
        datt = K.gemm(dx1, b.o_w, b_t=False, status=st)
        with self._fork(dx1, att):
            K.gemm(dx1, att, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=b.do_w,
                   split_k=K.wgrad_split(d, d, Mtok), status=st)
        dqkv = attention_bwd(datt, actx)
        with self._fork(dqkv, ln1):
            K.colsum_accum(dqkv, b.dqkv_b)
            K.gemm(dqkv, ln1, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=b.dqkv_w,
                   split_k=K.wgrad_split(3 * d, d, Mtok), status=st)
        dln1 = K.gemm(dqkv, b.qkv_w, b_t=False, status=st)
        return K.layernorm_bwd(dln1, x, b.ln1_w, mu1, rs1, b.dln1_w, b.dln1_b, dres=dx1, dres_sum=b.do_b)

    def _body_fwd(self, input_ids, hidden, keep: bool):
        if self.is_first:
            B, T = input_ids.shape
            x = self._embed(input_ids)
        else:
            B, T = hidden.shape[0], hidden.shape[1]
            x = hidden.reshape(B * T, -1)
            if x.dtype != BF16:
                x = x.to(BF16)
            x = x.contiguous()
        saved = []
        for b in self.blocks:
            x, s = self._block_fwd(b, x, B, T, keep)
            saved.append(s)
        return x, saved, B, T

    def _body_bwd(self, saved, dx: torch.Tensor, input_ids, B: int, T: int, sync: bool = False
                  ) -> Optional[torch.Tensor]:
        """``sync``: this is the step's last backward on this rank and the step ends with a gradient
        all-reduce, so every finished bucket is sent at once."""
        if sync and self.is_last:
            self._send_bucket()                       # final LayerNorm + LM head
        for b, s in zip(reversed(self.blocks), reversed(saved)):
            dx = self._block_bwd(b, s, dx)
            if sync:
                self._send_bucket()
        if self.is_first:
            K.embedding_bwd(input_ids.contiguous(), dx, self.dwte, self.dwpe)
            if sync:
                self._send_bucket()
            return None
        return dx.view(B, T, -1)

    # ------------------------------------------------------------------ engine API
    def forward(self, key: int, input_ids, hidden, keep: bool = True) -> torch.Tensor:
        x, saved, B, T = self._body_fwd(input_ids, hidden, keep)
        if keep:
            self.stash[key] = {"saved": saved, "ids": input_ids, "B": B, "T": T}
        return x.view(B, T, -1)

    def backward(self, key: int, grad_out: torch.Tensor, sync: bool = False) -> Optional[torch.Tensor]:
        s = self.stash.pop(key)
        B, T = s["B"], s["T"]
        dx = grad_out.reshape(B * T, -1)
        if dx.dtype != BF16:
            dx = dx.to(BF16)
        return self._body_bwd(s["saved"], dx.contiguous(), s["ids"], B, T, sync=self._want_overlap(sync))

    def _want_overlap(self, sync: bool) -> bool:
        return bool(sync and self._overlap and self.fused and self.world.num_replicas > 1)

    def _head(self, x: torch.Tensor, targets, mask, scale: float, grad: bool):
        """Final LayerNorm, LM head, masked CE.  Returns (loss, pieces for backward)."""
        lnf, mu, rs = K.layernorm_fwd(x, self.lnf_w, self.lnf_b)
        logits = K.gemm(lnf, self.head_w, status=self.status)
        loss = torch.zeros((), dtype=F32, device=x.device)
        K.cross_entropy(logits, targets.reshape(-1).contiguous(), mask.reshape(-1).contiguous() if mask is not None else None,
                        scale, loss, self.count_buf, write_grad=grad, status=self.status)
        return loss, (lnf, mu, rs, logits)

    def _head_chunked(self, x: torch.Tensor, targets, mask, scale: float, grad: bool):
        """The same head over ``train.lm_head_chunks`` slices of the token rows: logits, cross-entropy and (with
        ``grad``) the head's weight and input gradients of one slice before the next slice's logits exist
        (reference: the whole [tokens, vocabulary] tensor, src/model.py:146-147 and src/utils.py:184-193).
        Returns (loss, lnf, mean, rstd, dlnf or None)."""
        lnf, mu, rs = K.layernorm_fwd(x, self.lnf_w, self.lnf_b)
        M, d = lnf.shape
        V = self.head_w.shape[0]
        rows = -(-M // self.head_chunks)
        rows = -(-rows // 256) * 256                     # whole GEMM tiles per slice
        tg = targets.reshape(-1).contiguous()
        mk = mask.reshape(-1).contiguous() if mask is not None else None
        loss = torch.zeros((), dtype=F32, device=x.device)
        K.count_kept_rows(mk, M, self.count_buf)         # the mean is over the whole microbatch, not over a slice
        dlnf = torch.empty_like(lnf) if grad else None
        for r0 in range(0, M, rows):
            r1 = min(M, r0 + rows)
            logits = K.gemm(lnf[r0:r1], self.head_w, status=self.status)
            K.cross_entropy(logits, tg[r0:r1], mk[r0:r1] if mk is not None else None, scale, loss, self.count_buf,
                            write_grad=grad, status=self.status, count_ready=True)
            if grad:
                with self._fork(logits, lnf):
                    K.gemm(logits, lnf[r0:r1], a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=self.dhead_w,
                           split_k=K.wgrad_split(V, d, r1 - r0), status=self.status)
                K.gemm(logits, self.head_w, b_t=False, out=dlnf[r0:r1], status=self.status)
        return loss, lnf, mu, rs, dlnf

    def forward_backward(self, key: int, input_ids, hidden, targets, mask, scale: float, sync: bool = False):
        x, saved, B, T = self._body_fwd(input_ids, hidden, True)
        if self.head_chunks > 1:
            loss, lnf, mu, rs, dlnf = self._head_chunked(x, targets, mask, scale, grad=True)
        else:
            loss, (lnf, mu, rs, dlogits) = self._head(x, targets, mask, scale, grad=True)
            d = x.shape[1]
            V = dlogits.shape[1]
            with self._fork(dlogits, lnf):
                K.gemm(dlogits, lnf, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=self.dhead_w,
                       split_k=K.wgrad_split(V, d, x.shape[0]), status=self.status)
            dlnf = K.gemm(dlogits, self.head_w, b_t=False, status=self.status)
        dx = K.layernorm_bwd(dlnf, x, self.lnf_w, mu, rs, self.dlnf_w, self.dlnf_b)
        return loss, self._body_bwd(saved, dx, input_ids, B, T, sync=self._want_overlap(sync))

    @torch.no_grad()
    def forward_loss(self, input_ids, hidden, targets, mask, scale: float) -> torch.Tensor:
        x, _, _, _ = self._body_fwd(input_ids, hidden, False)
        if self.head_chunks > 1:
            return self._head_chunked(x, targets, mask, scale, grad=False)[0]
        loss, _ = self._head(x, targets, mask, scale, grad=False)
        return loss

    @torch.no_grad()
    def forward_infer(self, input_ids, hidden) -> torch.Tensor:
        x, _, B, T = self._body_fwd(input_ids, hidden, False)
        if self.is_last:
            lnf, _, _ = K.layernorm_fwd(x, self.lnf_w, self.lnf_b)
            x = K.gemm(lnf, self.head_w, status=self.status)
        return x.view(B, T, -1).float()

    # ------------------------------------------------------------------ sync + optimisers
    def sync_gradients(self) -> None:
        self._join()
        R = self.world.num_replicas
        if R == 1:
            return
        if self.fused:
            # buckets not sent during the last backward (none, if this rank had no microbatch) go now,
            # in the same order on every replica; then the compute stream waits for all of them
            while self._buckets_sent < len(self.buckets):
                self._send_bucket()
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            self._buckets_sent = 0
        else:
            dist.all_reduce(self.grad, group=self.world.curr_stage_group)
            self.grad.mul_(1.0 / R)

    def optimizer_step(self, lr: float, max_norm: float):
        self._join()
        K.grad_norm_and_clip(self.grad, self.stats, max_norm)
        self.opt_step += 1
        ic = self.inner_cfg
        if self.inner_type == "AdamW":
            K.adamw_step(self.theta, self.grad, self.m, self.v, self.w16, lr, ic.betas, ic.eps, ic.weight_decay,
                         self.opt_step, self.stats, zero_grad=True)
        else:
            K.sgd_step(self.theta, self.grad, self.mom_inner, self.w16, lr, ic.momentum if self.mom_inner is not None else 0.0,
                       ic.nesterov, self.stats, zero_grad=True)
        return self.stats[1]

    def outer_step(self, timer=None) -> None:
        """``timer`` (utils/timers.PhaseTimer): the wait for the slowest replica is recorded as phase
        "outer_wait", the synchronisation itself (fused kernel or library twin, plus the bf16 refresh of the
        weights) as "outer_sync", so that the second is the cost of the operation and not of the skew."""
        import contextlib
        phase = timer.phase if timer is not None else (lambda name: contextlib.nullcontext())
        with phase("outer_wait"):
            self.rendezvous.meet()        # absorbs the skew that H steps without contact have built up
        with phase("outer_sync"):
            self._outer_update()

    def _outer_update(self) -> None:
        o = self.outer
        if self.fused or o.R == 1:
            o.step()
        else:
            # library twin: NCCL all-reduce of the pseudo-gradient, then the update
            full_g = torch.empty(o.shard * o.R, dtype=F32, device=self.device)
            gathered = list(full_g.split(o.shard))
            dist.all_gather(gathered, o.theta_g, group=self.world.curr_stage_group)
            delta = full_g[:self.n] - self.theta
            dist.all_reduce(delta, group=self.world.curr_stage_group)
            delta.div_(o.R)
            d_sh = delta[o.lo:o.hi]
            mom = o.mom[:o.hi - o.lo]
            mom.mul_(o.mu).add_(d_sh)
            upd = d_sh + o.mu * mom if o.nesterov else mom
            o.theta_g[:o.hi - o.lo].sub_(o.lr * upd)
            dist.all_gather(gathered, o.theta_g, group=self.world.curr_stage_group)
            self.theta.copy_(full_g[:self.n])
        K.cast_to_bf16(self.theta, self.w16)

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {key: self.p32(key).detach().clone() for key, _, _ in self.specs}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for key, _, _ in self.specs:
            self.p32(key).copy_(sd[key])
        K.cast_to_bf16(self.theta, self.w16)

    def optim_state(self) -> dict:
        st = {"m": self.m.cpu(), "v": self.v.cpu(), "opt_step": self.opt_step}
        if self.mom_inner is not None:
            st["mom"] = self.mom_inner.cpu()
        return st

    def load_optim_state(self, st: dict) -> None:
        self.m.copy_(st["m"])
        self.v.copy_(st["v"])
        self.opt_step = int(st["opt_step"])
        if self.mom_inner is not None and "mom" in st:
            self.mom_inner.copy_(st["mom"])

    def outer_state(self) -> Optional[dict]:
        return self.outer.gather_state() if self.outer is not None else None

    def reset_outer(self) -> None:
        """Global weights := current weights, outer momentum := 0 (after loading weights that come
        without their DiLoCo state, e.g. a checkpoint moved to another topology)."""
        if self.outer is not None:
            self.outer.reset()

    def load_outer_state(self, st: Optional[dict]) -> None:
        if st is not None and self.outer is not None:
            self.outer.load_state(st)
