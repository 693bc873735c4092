"""Tensor-parallel batched decode of a BitNet-style model across the GPUs of one node (one process per GPU).

Partitioning (all splits are along output rows, in whole 64-row TL1 blocks and whole heads):

    q|k|v      rank r owns its query heads and their kv heads            -> local attention, local KV cache
    out proj   rank r owns hidden rows [r*h/R, (r+1)*h/R)
    gate|up    rank r owns ffn rows   [r*f/R, (r+1)*f/R) of both          -> ReLU^2*GLU stays local
    down       rank r owns hidden rows [r*h/R, (r+1)*h/R)
    LM head    rank r owns vocabulary rows [r*V/R, (r+1)*V/R)

After every sharded product the fp32 slices are all-gathered (NCCL over NVLink), so each rank runs the
*full-vector* RMSNorm + absmax quantiser in front of the next product exactly as a single GPU does:
same operation order, same int8 activations, and the integer products are exact. The token stream and
the logits are therefore bit-identical to the single-GPU engine (tests/test_gpu_tp.py checks that on
two GPUs). No floating-point reduction crosses ranks. The greedy argmax combines per-rank (max, index)
pairs and keeps the first maximum, as the reference's sampler does (TenzoEngine.cpp:1745-1755).

The per-kernel work goes through the library's C entry points (kernels.py); torch.distributed only
moves the slices. The kernels between two collectives are replayed as one CUDA graph; the collectives are direct calls.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import abi


@dataclass(frozen=True)
class TPPlan:
    """Row ranges (in elements) one rank owns; everything is validated to be whole blocks / heads."""
    world: int
    rank: int
    q_heads: tuple       # (first, count)
    kv_heads: tuple
    hidden_rows: tuple
    ffn_rows: tuple
    vocab_rows: tuple


def plan(cfg: dict, world: int, rank: int) -> TPPlan:
    """Partition of `cfg` (hidden_size, ffn_dim, num_q_heads, num_kv_heads, head_dim, vocab_size) for `rank` of `world`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    h, f, nq, nkv, hd, v = (cfg[k] for k in ("hidden_size", "ffn_dim", "num_q_heads", "num_kv_heads", "head_dim", "vocab_size"))
    if hd != 128:
        raise ValueError("head_dim must be 128")
    if nkv % world or nq % nkv:
        raise ValueError(f"{nkv} kv heads do not split across {world} ranks")
    if h % (64 * world) or f % (64 * world):
        raise ValueError("hidden_size and ffn_dim must split into whole 64-row blocks per rank")
    if v % (4 * world):
        raise ValueError("vocab_size must be a multiple of 4 * world")
    kv_loc, q_loc = nkv // world, nq // world
    return TPPlan(world, rank, (rank * q_loc, q_loc), (rank * kv_loc, kv_loc), (rank * h // world, h // world),
                  (rank * f // world, f // world), (rank * v // world, v // world))


def combine_argmax(vals, idxs):
    """vals, idxs: [world, batch] per-rank maxima and their global vocabulary indices (rank r's indices all lie below
    rank r+1's). Returns [batch] indices of the first maximum: larger value, ties to the lower rank."""
    import torch
    best = vals.max(dim=0).values
    first_rank = (vals == best.unsqueeze(0)).to(torch.int32).argmax(dim=0)      # argmax returns the first maximal entry
    return idxs.gather(0, first_rank.unsqueeze(0)).squeeze(0)


def all_gather_cols(loc, full, scratch, world: int, group=None):
    """full[:, r*S:(r+1)*S] = rank r's `loc` ([B, S] on every rank). `scratch` holds at least world*B*S elements."""
    if world == 1:
        full.copy_(loc)
        return
    import torch.distributed as dist
    B, S = loc.shape
    tmp = scratch[: world * B * S].view(world, B, S)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(tmp, loc, group=group)
    else:                                                   # gloo (CPU tests) has no single-tensor all-gather
        dist.all_gather(list(tmp.unbind(0)), loc.contiguous(), group=group)
    full.view(B, world, S).copy_(tmp.transpose(0, 1))


def _tl1_rows(w: np.ndarray, n: int, k: int, r0: int, cnt: int) -> np.ndarray:
    """Rows [r0, r0+cnt) of a TL1-packed [n x k] matrix (whole 64-row blocks are contiguous in the packing)."""
    assert r0 % 64 == 0 and cnt % 64 == 0
    return np.ascontiguousarray(w.reshape(n // 64, -1)[r0 // 64:(r0 + cnt) // 64]).reshape(-1)


class TensorParallelDecoder:
    """Greedy batched decode with the weights of `model` (synth.SyntheticModel-like: .cfg, .layers, .final_norm,
    .lm_w, .lm_scales) sharded as in `plan`. `group` is a torch.distributed process group (None: the default)."""

    def __init__(self, model, batch: int, max_seq: int, group=None, rope_theta: float = 10000.0, use_graph: bool | None = None):
        """`model`: a synth.SyntheticModel-like object, or a plain config dict (then call load_random).
        `use_graph`: replay the kernels between two collectives as CUDA graphs (default) instead of launching them one
        by one. The NCCL calls stay outside the graphs: capturing them together with the kernels did not complete on
        the test machines (the first replay never returned)."""
        import torch
        import torch.distributed as dist
        from . import kernels, load_library
        self.torch, self.dist, self.k, self.group = torch, dist, kernels, group
        self.lib = load_library()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        cfg = self.cfg = dict(model if isinstance(model, dict) else model.cfg)
        self.p = p = plan(cfg, self.world, self.rank)
        self.B, self.max_seq = batch, max_seq
        self.use_graph = True if use_graph is None else bool(use_graph)
        h, f, hd = cfg["hidden_size"], cfg["ffn_dim"], cfg["head_dim"]
        nq, nkv = cfg["num_q_heads"], cfg["num_kv_heads"]
        self.dev = dev = torch.device("cuda", torch.cuda.current_device())
        qn, kn = p.q_heads[1] * hd, p.kv_heads[1] * hd
        v0, vn = p.vocab_rows
        self.layers = []
        if not isinstance(model, dict):
            self._load_model(model)
        L = cfg["num_layers"]
        kv_loc = p.kv_heads[1]
        self.ck = torch.zeros(batch, L, kv_loc, max_seq, hd, dtype=torch.int8, device=dev)
        self.cv = torch.zeros_like(self.ck)
        self.sk = torch.zeros(batch, L, kv_loc, max_seq, dtype=torch.float32, device=dev)
        self.sv = torch.zeros_like(self.sk)
        cs, sn = np.zeros((max_seq, hd // 2), np.float32), np.zeros((max_seq, hd // 2), np.float32)
        rc = self.lib.tenzo_ext_rope_tables(max_seq, hd, rope_theta, cs.ctypes.data_as(abi.c_f32p), sn.ctypes.data_as(abi.c_f32p))
        if rc != 0:
            raise RuntimeError("tenzo_ext_rope_tables failed")
        self.rope_cos, self.rope_sin = torch.from_numpy(cs).to(dev), torch.from_numpy(sn).to(dev)
        self.pos = torch.zeros(batch, dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        R, B = self.world, batch
        self.b_qkv = torch.empty(B, qn + 2 * kn, **f32)
        self.b_attn_loc = torch.empty(B, qn, **f32)
        self.b_attn = torch.empty(B, nq * hd, **f32)
        self.b_h1_loc, self.b_h1 = torch.empty(B, h // R, **f32), torch.empty(B, h, **f32)
        self.b_act_loc, self.b_act = torch.empty(B, f // R, **f32), torch.empty(B, f, **f32)
        self.b_x_loc, self.b_x = torch.empty(B, h // R, **f32), torch.empty(B, h, **f32)
        self.b_gather = torch.empty(R * B * max(nq * hd, f, h) // R, **f32)
        self.ws = torch.empty(self.lib.tenzo_cuda_tl1_gemv_workspace_bytes(B, max(h, f, nq * hd)), dtype=torch.uint8, device=dev)
        self.tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.next_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.logits_loc = torch.empty(B, vn, **f32)
        self.prog, self.graphs = None, None
        self.collectives_per_step = (4 * L + 2) if self.world > 1 else 0
        self.kernels_per_step = 5 * L + 4      # TL1 x4 (+ quantiser when batched) and attention per layer; embedding, LM head (+ quantiser, argmax)

    def _load_model(self, model):
        torch, p, cfg = self.torch, self.p, self.cfg
        h, f, hd, nq, nkv = cfg["hidden_size"], cfg["ffn_dim"], cfg["head_dim"], cfg["num_q_heads"], cfg["num_kv_heads"]
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)
        q0, qn = p.q_heads[0] * hd, p.q_heads[1] * hd
        k0, kn = p.kv_heads[0] * hd, p.kv_heads[1] * hd
        for lw in model.layers:
            d = {}
            d["qkv"] = up(np.concatenate([_tl1_rows(lw["q_w"], nq * hd, h, q0, qn), _tl1_rows(lw["k_w"], nkv * hd, h, k0, kn),
                                          _tl1_rows(lw["v_w"], nkv * hd, h, k0, kn)]))
            d["qkv_scales"] = [float(lw["q_scale"]), float(lw["k_scale"]), float(lw["v_scale"])]
            d["o"] = up(_tl1_rows(lw["out_w"], h, nq * hd, *p.hidden_rows))
            d["o_scale"] = float(lw["out_scale"])
            d["gu"] = up(np.concatenate([_tl1_rows(lw["gate_w"], f, h, *p.ffn_rows), _tl1_rows(lw["up_w"], f, h, *p.ffn_rows)]))
            d["gu_scales"] = [float(lw["gate_scale"]), float(lw["up_scale"])]
            d["down"] = up(_tl1_rows(lw["down_w"], h, f, *p.hidden_rows))
            d["down_scale"] = float(lw["down_scale"])
            for n in ("in_norm", "attn_sub_norm", "post_norm", "ffn_sub_norm"):
                d[n] = up(lw[n])
            self.layers.append(d)
        self.final_norm = up(model.final_norm)
        v0, vn = p.vocab_rows
        self.lm_w, self.lm_s = up(model.lm_w[v0:v0 + vn]), up(model.lm_scales[v0:v0 + vn])
        self.emb_w, self.emb_s = up(model.lm_w), up(model.lm_scales)      # tied embedding, replicated: a lookup touches one row

    def load_random(self, seed: int = 0, context: int = 0):
        """Seeded random shards generated on the device (i.i.d. ternary TL1 bytes, int8 LM head rows; the embedding
        table uses a seed common to all ranks) and, if `context` > 0, a KV cache pre-filled to that length with random
        int8 rows. For measurements at shapes whose host-side generation would take minutes; not for parity checks."""
        from . import synth
        torch, p, cfg = self.torch, self.p, self.cfg
        h, f, hd, nq = cfg["hidden_size"], cfg["ffn_dim"], cfg["head_dim"], cfg["num_q_heads"]
        qn, kn = p.q_heads[1] * hd, p.kv_heads[1] * hd
        g = torch.Generator(device=self.dev).manual_seed(1000 * seed + self.rank)
        table = torch.from_numpy(synth._BYTE81).to(self.dev)
        tl1 = lambda rows, k: table[torch.randint(0, 81, (rows * k // 4,), generator=g, device=self.dev)].contiguous()
        norm = lambda n, gs: 1.0 + 0.1 * torch.randn(n, generator=gs, device=self.dev)
        self.layers = []
        for l in range(cfg["num_layers"]):
            gs = torch.Generator(device=self.dev).manual_seed(77 * seed + l)         # replicated tensors: same on every rank
            self.layers.append(dict(qkv=tl1(qn + 2 * kn, h), qkv_scales=[0.016, 0.016, 0.016], o=tl1(p.hidden_rows[1], nq * hd), o_scale=0.016,
                                    gu=tl1(2 * p.ffn_rows[1], h), gu_scales=[0.016, 0.016], down=tl1(p.hidden_rows[1], f), down_scale=0.016,
                                    in_norm=norm(h, gs), attn_sub_norm=norm(nq * hd, gs), post_norm=norm(h, gs), ffn_sub_norm=norm(f, gs)))
        gs = torch.Generator(device=self.dev).manual_seed(77 * seed + 9999)
        self.final_norm = norm(h, gs)
        v = cfg["vocab_size"]
        self.emb_w = torch.randint(-127, 128, (v, h), generator=gs, device=self.dev, dtype=torch.int8)
        self.emb_s = 0.0005 + 0.0005 * torch.rand(v, generator=gs, device=self.dev)
        v0, vn = p.vocab_rows
        self.lm_w, self.lm_s = self.emb_w[v0:v0 + vn].contiguous(), self.emb_s[v0:v0 + vn].contiguous()
        if context > 0:
            assert context < self.max_seq
            self.ck[:, :, :, :context].copy_(torch.randint(-127, 128, self.ck[:, :, :, :context].shape, generator=g, device=self.dev, dtype=torch.int8))
            self.cv[:, :, :, :context].copy_(torch.randint(-127, 128, self.cv[:, :, :, :context].shape, generator=g, device=self.dev, dtype=torch.int8))
            self.sk[:, :, :, :context] = 0.01 + 0.02 * torch.rand(self.sk[:, :, :, :context].shape, generator=g, device=self.dev)
            self.sv[:, :, :, :context] = 0.01 + 0.02 * torch.rand(self.sv[:, :, :, :context].shape, generator=g, device=self.dev)
            self.pos.fill_(context)
        return self

    # ---- one token for every sequence ---------------------------------------------------------------
    def _program(self):
        """The step as a list of ("compute", fn) and ("comm", fn) items: compute items only launch kernels on the
        current stream (capturable), comm items are the NCCL all-gathers between them."""
        k, p, cfg, torch, dist = self.k, self.p, self.cfg, self.torch, self.dist
        h, f, hd = cfg["hidden_size"], cfg["ffn_dim"], cfg["head_dim"]
        qn, kn = p.q_heads[1] * hd, p.kv_heads[1] * hd
        h0, hn = p.hidden_rows
        fn = p.ffn_rows[1]
        R, B = self.world, self.B
        prog = []

        def gather(loc, full):
            """comm: slices -> scratch [R][B][S]; the following compute item starts by transposing them into `full`."""
            S = loc.shape[1]
            tmp = self.b_gather[: R * B * S].view(R, B, S)
            if R > 1:
                prog.append(("comm", lambda: dist.all_gather_into_tensor(tmp, loc, group=self.group)))
                return lambda: full.view(B, R, S).copy_(tmp.transpose(0, 1))
            return lambda: full.copy_(loc)

        def embed():
            x = k.embedding_i8(self.emb_w, self.emb_s, self.tokens)                  # [B, h], identical on every rank
            self.b_x.copy_(x)
            self.b_x_loc.copy_(self.b_x[:, h0:h0 + hn])
        pending = [embed]
        assert len(self.layers) == cfg["num_layers"], "no weights loaded"
        for l, d in enumerate(self.layers):
            nb = (qn + 2 * kn) // 64

            def attn_block(l=l, d=d, nb=nb):
                k.tl1_gemv(self.b_x, d["qkv"], nb, h, d["qkv_scales"], [qn // 64, (qn + kn) // 64, nb], norm_w=d["in_norm"], do_norm=True,
                           out=self.b_qkv, workspace=self.ws)
                k.attention_int8(self.b_qkv[:, :qn], self.b_qkv[:, qn:qn + kn], self.b_qkv[:, qn + kn:], self.ck, self.cv, self.sk, self.sv,
                                 self.pos, layer=l, n_q=p.q_heads[1], n_kv=p.kv_heads[1], max_seq=self.max_seq, rope_cos=self.rope_cos,
                                 rope_sin=self.rope_sin, max_len=self.max_seq, out=self.b_attn_loc)
            pending.append(attn_block)
            prog.append(("compute", pending))
            pending = [gather(self.b_attn_loc, self.b_attn)]
            pending.append(lambda d=d: k.tl1_gemv(self.b_attn, d["o"], hn // 64, cfg["num_q_heads"] * hd, [d["o_scale"]], norm_w=d["attn_sub_norm"],
                                                  do_norm=True, epilogue=k.EPI_RESIDUAL, resid=self.b_x_loc, out=self.b_h1_loc, workspace=self.ws))
            prog.append(("compute", pending))
            pending = [gather(self.b_h1_loc, self.b_h1)]
            pending.append(lambda d=d: k.tl1_gemv(self.b_h1, d["gu"], 2 * fn // 64, h, d["gu_scales"], [fn // 64, 2 * fn // 64, 2 * fn // 64],
                                                  norm_w=d["post_norm"], do_norm=True, epilogue=k.EPI_RELU2_GLU, out=self.b_act_loc, workspace=self.ws))
            prog.append(("compute", pending))
            pending = [gather(self.b_act_loc, self.b_act)]
            pending.append(lambda d=d: k.tl1_gemv(self.b_act, d["down"], hn // 64, f, [d["down_scale"]], norm_w=d["ffn_sub_norm"], do_norm=True,
                                                  epilogue=k.EPI_RESIDUAL, resid=self.b_h1_loc, out=self.b_x_loc, workspace=self.ws))
            prog.append(("compute", pending))
            pending = [gather(self.b_x_loc, self.b_x)]

        vals = torch.empty(R, B, dtype=torch.float32, device=self.dev)
        idxs = torch.empty(R, B, dtype=torch.int32, device=self.dev)
        val_loc = torch.empty(B, dtype=torch.float32, device=self.dev)
        idx_loc = torch.empty(B, dtype=torch.int32, device=self.dev)

        def head():
            self.pos.add_(1)
            _, _, arg = k.lm_head_i8(self.b_x, self.lm_w, self.lm_s, norm_w=self.final_norm, logits=self.logits_loc)
            val_loc.copy_(self.logits_loc.gather(1, arg.to(torch.int64).unsqueeze(1)).squeeze(1))
            idx_loc.copy_(arg + p.vocab_rows[0])
        pending.append(head)
        prog.append(("compute", pending))
        if R > 1:
            prog.append(("comm", lambda: (dist.all_gather_into_tensor(vals, val_loc, group=self.group),
                                          dist.all_gather_into_tensor(idxs, idx_loc, group=self.group))))
            prog.append(("compute", [lambda: self.next_tokens.copy_(combine_argmax(vals, idxs.to(torch.int64)).to(torch.int32))]))
        else:
            prog.append(("compute", [lambda: self.next_tokens.copy_(idx_loc)]))
        # merge neighbouring compute items
        merged = []
        for kind, item in prog:
            if kind == "compute" and merged and merged[-1][0] == "compute":
                merged[-1][1].extend(item)
            else:
                merged.append((kind, list(item) if kind == "compute" else item))
        return merged

    def _run_eager(self, prog):
        for kind, item in prog:
            if kind == "compute":
                for fn in item:
                    fn()
            else:
                item()

    def step(self, tokens=None):
        """Feed one token per sequence (device or host int32 [B]; None: the previous step's argmax) and return the
        device tensor of next tokens (valid after the stream reaches this point). With `use_graph` every run of
        kernels between two collectives is one CUDA graph; the collectives themselves are issued directly."""
        torch = self.torch
        if tokens is None:
            self.tokens.copy_(self.next_tokens)
        else:
            self.tokens.copy_(torch.as_tensor(tokens, dtype=torch.int32).to(self.tokens.device, non_blocking=True))
        if self.prog is None:
            self.prog = self._program()
        if not self.use_graph:
            self._run_eager(self.prog)
            return self.next_tokens
        if self.graphs is None:
            pos0 = self.pos.clone()
            self._run_eager(self.prog)      # warm-up outside capture (function attributes, NCCL channels); the cache row it
            torch.cuda.synchronize()        # appends at pos0 is rewritten with the same bytes by the captured step
            self.pos.copy_(pos0)
            self.graphs, pool = [], None
            for kind, item in self.prog:
                if kind != "compute":
                    self.graphs.append(None)
                    continue
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool):
                    for fn in item:
                        fn()
                pool = pool or g.pool()
                self.graphs.append(g)
        for (kind, item), g in zip(self.prog, self.graphs):
            if g is not None:
                g.replay()
            else:
                item()
        return self.next_tokens

    def logits_slice(self):
        """This rank's [B, V/R] logits of the last step."""
        return self.logits_loc


def parity_check(group=None, use_graph: bool = True, say=None) -> bool:
    """The tensor-parallel decoder next to the single-GPU engine on one seeded model (the synthetic 8B shape cut to 2 layers
    and a 16384-row vocabulary; 32 sequences, 3 prompt tokens + 6 greedy steps), on the process group that is already
    initialised (or a single process). True when, on every rank, the token streams are identical and this rank's slice of
    the last step's logits equals the engine's bits for the first and the last sequence. Collective: every rank of the
    group must call it."""
    import torch
    import torch.distributed as dist
    from . import synth
    from .engine import Engine
    say = say or (lambda m: None)
    cfg = dict(synth.SYNTH_8B, num_layers=2, vocab_size=16384, max_seq_len=64)
    B, prompt_len, steps = 32, 3, 6
    model = synth.SyntheticModel(cfg, seed=5)
    prompts = np.stack([synth.prompt_tokens(100 + b, prompt_len, cfg["vocab_size"]) for b in range(B)])     # [B, prompt_len]
    say("model built")
    eng = Engine(model.config_struct(), batch=B).load_synthetic(model)
    for t in range(prompt_len - 1):
        eng.prefill_tokens(prompts[:, t])
    want = eng.decode_greedy(prompts[:, -1], steps - 1)                   # [steps - 1, B]
    last = eng.generate_steps(want[-1])                                   # the last step also leaves its logits behind
    want = np.concatenate([want, np.asarray(last)[None]])
    want_logits = np.stack([eng.read_buffer(15, seq=b, count=cfg["vocab_size"]) for b in (0, B - 1)])
    eng.close()
    say("single-GPU engine done")
    dec = TensorParallelDecoder(model, B, cfg["max_seq_len"], group=group, use_graph=use_graph)
    say("shards loaded")
    for t in range(prompt_len - 1):
        dec.step(prompts[:, t])
        torch.cuda.synchronize()
    got = []
    nxt = dec.step(prompts[:, -1])
    got.append(nxt.cpu().numpy().copy())
    for _ in range(steps - 1):
        nxt = dec.step()
        got.append(nxt.cpu().numpy().copy())
    got = np.stack(got)
    say("decode done")
    v0, vn = dec.p.vocab_rows
    mine = dec.logits_slice().cpu().numpy()
    ok = bool(np.array_equal(got, want) and np.array_equal(mine[0], want_logits[0, v0:v0 + vn]) and
              np.array_equal(mine[B - 1], want_logits[1, v0:v0 + vn]))
    if not ok:
        say(f"MISMATCH: tokens equal={np.array_equal(got, want)}, first differing step={np.argwhere(got != want)[:1].tolist()}")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        ok = bool(flag.item())
    del dec
    torch.cuda.empty_cache()
    return ok
