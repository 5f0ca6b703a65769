"""Tensor-parallel OPT decoder over R-sharded BSI linears, for one node with several GPUs.

Every BSI linear keeps only its own block of output rows (keys), as `BSIShardedLinear` does, but the
activations travel between the ranks in their packed form and nothing is computed twice:

* the residual stream is sharded by tokens: rank g owns rows [g*Q/G, (g+1)*Q/G) of the [Q, H]
  hidden states and does the residual adds, both LayerNorms and the activation packing for them;
* q/k/v are one fused key set holding the rows of the rank's own attention heads, so attention runs
  on local heads with no exchange;
* what the ranks exchange are the int8 images and chunk scales of the packed activations (half the
  bytes of the fp16 values, a quarter of fp32): an all-gather along the token axis after each
  LayerNorm, an all-gather along the feature axis after attention and after fc1 (chunk scales cover
  256 consecutive features, so a rank can quantise its own feature block on its own), and an
  all-to-all that turns the [Q, H/G] outputs of out_proj / fc2 back into token shards.

Per output element the arithmetic is that of the single-GPU layer (same chunk quantisation, same
integer dot, same float32 chunk combine, same cast + bias), so G ranks reproduce the 1-GPU hidden
states bit for bit; G = 1 skips every collective and is the fused single-GPU forward (one QKV
launch, ReLU inside the fc1 epilogue).

The reference has no distributed code; the layer arithmetic follows its BSIQuantizedLinear
(bsi_ops/benchmarks/verify_accuracy_bsi.py:46-215) and the OPT wiring of
benchmark_performance_bsi.py.

With the CUDA extension and more than one rank the exchanges are not library collectives: every rank
owns a peer-mapped buffer (CUDA IPC), the pack kernel stores its int8 image and scales into the
buffers of all ranks at once, the out_proj / fc2 epilogue stores each output row into the buffer of
the rank that owns the token (`PeerExchange`), and a bounded flag barrier separates writers from
readers. `exchange="collective"` keeps NCCL / gloo all-gathers and all-to-alls (what the CPU tests run).

`ops` carries the three device operations (key build, activation pack, packed linear); the CPU
tests drive the same orchestration over gloo with stand-ins.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .opt import CONFIGS, OPTConfig


class BsiDeviceOps:
    """The three BSI operations of a tensor-parallel layer, on the CUDA extension."""

    def __init__(self, decimal_places: int = 2, compress_threshold: float = 0.5):
        from . import bsi_ops  # fails loudly when the extension is missing

        self.m = bsi_ops
        self.dp = int(decimal_places)
        self.threshold = float(compress_threshold)

    def build_keys(self, weight: torch.Tensor):
        cap, mem, num_keys, d, w = self.m.build_bsi_keys_cuda(weight.float(), self.dp, self.threshold)
        return cap

    def pack_into(self, x2d, q8, scales):
        self.m.pack_queries_into(x2d, q8, scales, self.dp)

    def linear(self, q8, scales, keys, bias, out_dtype, relu=False):
        return self.m.linear_from_packed(q8, scales, keys, bias, self.dp, out_dtype, relu)

    def add_ln_pack(self, x, delta, ln, q8_ptrs, ld8, scale_ptrs, scale_ld):
        """x + delta (delta may be None), LayerNorm `ln` of the sum, packed to the given addresses; returns the sum."""
        return self.m.add_layernorm_pack(x, delta, ln.weight, ln.bias, ln.eps, q8_ptrs, ld8, scale_ptrs, scale_ld, self.dp)

    def linear_requant(self, q8, scales, keys, bias, layer_dtype, relu, q8_ptrs, ld8, scale_ptrs, scale_ld):
        """Linear whose output is re-quantised for the next linear inside its epilogue and stored to the given
        addresses (needs a 16-bit layer type and a multiple of 256 output features)."""
        self.m.linear_from_packed_requant(q8, scales, keys, bias, self.dp, layer_dtype, relu, q8_ptrs, ld8,
                                          scale_ptrs, scale_ld)


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class PeerExchange:
    """One rank's peer-mapped exchange buffers for a fixed batch shape, and the barrier between phases.

    Regions (every rank has the same layout; peers write, the owner reads):
      R   packed activations of all tokens after a LayerNorm      q8 [Q, H],  scales [Q, H/256]
      C1  packed attention output of all tokens                    q8 [Q, H],  scales [Q, H/256]
      C2  packed fc1 output of all tokens                          q8 [Q, F],  scales [Q, F/256]
      T   out_proj / fc2 outputs of the rank's own tokens          [Q/G, H] in the model dtype
    A region is rewritten only after at least one barrier that follows its last reader on every rank,
    so one copy of each is enough."""

    def __init__(self, m, rank, world, group, Q, H, Fd, dtype, device, timeout_ms=30000):
        self.m, self.rank, self.world, self.timeout_ms = m, rank, world, int(timeout_ms)
        self.Q, self.H, self.F, self.Qn = Q, H, Fd, Q // world
        esz = torch.empty(0, dtype=dtype).element_size()
        self.esz = esz
        sizes = [("flags", 256), ("R_q8", Q * H), ("R_sc", Q * (H // 256) * 4), ("C1_q8", Q * H),
                 ("C1_sc", Q * (H // 256) * 4), ("C2_q8", Q * Fd), ("C2_sc", Q * (Fd // 256) * 4),
                 ("T", self.Qn * H * esz)]
        self.off, total = {}, 0
        for name, n in sizes:
            self.off[name] = total
            total += _align(n)
        self.buf, handle = m.peer_alloc(total)
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        self.base = [self.buf.data_ptr() if r == rank else m.peer_open(handles[r]) for r in range(world)]

        def view(name, shape, dt):
            n = 1
            for d in shape:
                n *= d
            nbytes = n * torch.empty(0, dtype=dt).element_size()
            return self.buf[self.off[name]:self.off[name] + nbytes].view(dt).view(*shape)

        self.R_q8, self.R_sc = view("R_q8", (Q, H), torch.int8), view("R_sc", (Q, H // 256), torch.float32)
        self.C1_q8, self.C1_sc = view("C1_q8", (Q, H), torch.int8), view("C1_sc", (Q, H // 256), torch.float32)
        self.C2_q8, self.C2_sc = view("C2_q8", (Q, Fd), torch.int8), view("C2_sc", (Q, Fd // 256), torch.float32)
        self.T = view("T", (self.Qn, H), dtype)
        dist.barrier(group=group)   # every rank has mapped every buffer before anyone writes

    def ptrs(self, name, byte_offset=0):
        """Address of region `name` (+ byte_offset) in every rank's buffer, as seen from this process."""
        return [b + self.off[name] + byte_offset for b in self.base]

    def pack_to_all(self, x, dp, q8_name, sc_name, q8_off, sc_off, ld8, scale_ld, height):
        """Packs x and leaves its int8 image at byte offset q8_off of region q8_name (row pitch ld8) and its
        chunk scales at byte offset sc_off of sc_name (scale_ld floats per row) on every rank -- the pack kernel
        stores each packed unit to all of them -- then passes the barrier."""
        q8_ptrs, sc_ptrs = self.ptrs(q8_name, q8_off), self.ptrs(sc_name, sc_off)
        g, G = self.rank, self.world
        # the kernel walks its destinations in list order: start each rank at its successor, so that at any
        # moment the ranks write to different peers instead of all converging on the same one
        order = [(g + 1 + k) % G for k in range(G)]
        self.m.pack_queries_multi(x, [q8_ptrs[r] for r in order], ld8, [sc_ptrs[r] for r in order], scale_ld, dp)
        self.barrier()

    def barrier(self):
        self.m.peer_barrier(self.ptrs("flags"), self.rank, self.timeout_ms)

    def close(self):
        for r, b in enumerate(self.base):
            if r != self.rank:
                self.m.peer_close(b)
        self.base = []


def _block(n: int, world: int, rank: int, multiple: int, what: str):
    if n % (world * multiple) != 0:
        raise ValueError(f"{what}={n} must be a multiple of {world} ranks x {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


class TPDecoderLayer(nn.Module):
    """One OPT decoder layer on rank `rank` of `world`; see the module docstring for the data flow."""

    def __init__(self, cfg: OPTConfig, rank, world, group, ops, dtype, device, fuse_ln=False):
        super().__init__()
        self.cfg, self.rank, self.world, self.group, self.ops, self.dtype = cfg, rank, world, group, ops, dtype
        H, Fd = cfg.hidden_size, cfg.ffn_dim
        self.head_dim = H // cfg.num_attention_heads
        if cfg.num_attention_heads % world != 0:
            raise ValueError("attention heads must divide evenly over the ranks")
        self.h_lo, self.h_hi = _block(H, world, rank, 256 if world > 1 else 1, "hidden_size")
        self.f_lo, self.f_hi = _block(Fd, world, rank, 256 if world > 1 else 1, "ffn_dim")
        self.local_heads = cfg.num_attention_heads // world
        # fc1 -> ReLU -> re-quantise inside the fc1 epilogue: CUDA extension, 16-bit layer type, whole chunks per rank
        self.fuse_requant = (isinstance(ops, BsiDeviceOps) and dtype in (torch.float16, torch.bfloat16)
                             and (self.f_hi - self.f_lo) % 256 == 0 and ops.dp <= 3)
        # residual add + LayerNorm + pack in one kernel (CUDA extension, 16-bit layer type): opt-in. Its float32
        # mean / variance are summed in another order than torch's LayerNorm, so about one packed integer in a
        # million differs from torch LayerNorm -> pack; through the re-quantisations of the following layers that is
        # enough to move 3 % of the next-token argmaxes of a random-init OPT-125M (measured), so the default keeps
        # torch's LayerNorm and stays bit-identical to the reference's layer flow.
        self.fuse_ln = (bool(fuse_ln) and isinstance(ops, BsiDeviceOps) and dtype in (torch.float16, torch.bfloat16)
                        and H % 256 == 0 and H <= 16384)
        self.self_attn_layer_norm = nn.LayerNorm(H, device=device, dtype=dtype)
        self.final_layer_norm = nn.LayerNorm(H, device=device, dtype=dtype)
        self.keys_qkv = self.keys_out = self.keys_fc1 = self.keys_fc2 = None
        self.bias_qkv = self.bias_out = self.bias_fc1 = self.bias_fc2 = None

    # -- construction ----------------------------------------------------------------------------
    @torch.no_grad()
    def load_linears(self, weights: dict, biases: dict):
        """weights / biases: full (unsharded) tensors by HF name (q_proj ... fc2); the rank keeps its rows."""
        hs = slice(self.h_lo, self.h_hi)
        fs = slice(self.f_lo, self.f_hi)
        wqkv = torch.cat([weights["q_proj"][hs], weights["k_proj"][hs], weights["v_proj"][hs]], dim=0)
        self.keys_qkv = self.ops.build_keys(wqkv)
        self.keys_out = self.ops.build_keys(weights["out_proj"][hs])
        self.keys_fc1 = self.ops.build_keys(weights["fc1"][fs])
        self.keys_fc2 = self.ops.build_keys(weights["fc2"][hs])
        f32 = lambda t: t.detach().float().contiguous()
        self.bias_qkv = f32(torch.cat([biases["q_proj"][hs], biases["k_proj"][hs], biases["v_proj"][hs]]))
        self.bias_out = f32(biases["out_proj"][hs])
        self.bias_fc1 = f32(biases["fc1"][fs])
        self.bias_fc2 = f32(biases["fc2"][hs])

    # -- exchanges -------------------------------------------------------------------------------
    def _pack_gather_rows(self, h_loc, Q):
        """h_loc [Q/G, D] (own tokens) -> packed activations of all tokens: q8 [Q, D], scales [Q, D/256]."""
        Qn, D = h_loc.shape
        if self.world == 1:
            q8 = torch.empty(Q, D, dtype=torch.int8, device=h_loc.device)
            sc = torch.empty(Q, D // 256, dtype=torch.float32, device=h_loc.device)
            self.ops.pack_into(h_loc, q8, sc)
            return q8, sc
        q8_loc = torch.empty(Qn, D, dtype=torch.int8, device=h_loc.device)
        sc_loc = torch.empty(Qn, D // 256, dtype=torch.float32, device=h_loc.device)
        self.ops.pack_into(h_loc, q8_loc, sc_loc)
        q8 = torch.empty(Q, D, dtype=torch.int8, device=h_loc.device)
        sc = torch.empty(Q, D // 256, dtype=torch.float32, device=h_loc.device)
        dist.all_gather_into_tensor(q8, q8_loc, group=self.group)      # rank-major along dim 0 = token order
        dist.all_gather_into_tensor(sc, sc_loc, group=self.group)
        return q8, sc

    def _pack_gather_cols(self, y_loc):
        """y_loc [Q, D/G] (own features of all tokens) -> q8 [Q, D], scales [Q, D/256]."""
        Q, Dl = y_loc.shape
        G = self.world
        q8_loc = torch.empty(Q, Dl, dtype=torch.int8, device=y_loc.device)
        sc_loc = torch.empty(Q, Dl // 256, dtype=torch.float32, device=y_loc.device)
        self.ops.pack_into(y_loc, q8_loc, sc_loc)
        if G == 1:
            return q8_loc, sc_loc
        q8_all = torch.empty(G * Q, Dl, dtype=torch.int8, device=y_loc.device)
        sc_all = torch.empty(G * Q, Dl // 256, dtype=torch.float32, device=y_loc.device)
        dist.all_gather_into_tensor(q8_all, q8_loc, group=self.group)
        dist.all_gather_into_tensor(sc_all, sc_loc, group=self.group)
        q8 = q8_all.view(G, Q, Dl).permute(1, 0, 2).reshape(Q, G * Dl).contiguous()
        sc = sc_all.view(G, Q, Dl // 256).permute(1, 0, 2).reshape(Q, G * (Dl // 256)).contiguous()
        return q8, sc

    def _to_token_shard(self, o):
        """o [Q, H/G] (own output features of all tokens) -> [Q/G, H] (all features of own tokens)."""
        G = self.world
        if G == 1:
            return o
        Q, Rl = o.shape
        recv = torch.empty_like(o)
        dist.all_to_all_single(recv, o.contiguous(), group=self.group)   # block p of recv: rank p's features, my tokens
        return recv.view(G, Q // G, Rl).permute(1, 0, 2).reshape(Q // G, G * Rl)

    # -- forward ---------------------------------------------------------------------------------
    def _attention(self, qkv, B, T):
        Hl, nh, hd = self.h_hi - self.h_lo, self.local_heads, self.head_dim
        q, k, v = (qkv[:, i * Hl:(i + 1) * Hl].view(B, T, nh, hd).transpose(1, 2) for i in range(3))
        # query scaled in the model's type, attention with unit scaling: the order HuggingFace's OPT uses
        attn = F.scaled_dot_product_attention(q * hd ** -0.5, k, v, is_causal=True, scale=1.0)   # [B, nh, T, hd]
        return attn.transpose(1, 2).reshape(B * T, Hl)

    def forward_peer(self, x_loc, delta, B, T, px: "PeerExchange"):
        """The layer with stores into peer buffers in place of collectives (see PeerExchange). `delta` is the
        previous layer's fc2 output for the own tokens, still to be added to the residual stream (None at the
        first layer); returns (x, delta) in the same form."""
        ops, dt, m, g = self.ops, self.dtype, self.ops.m, self.rank
        H, Fd, Qn = self.cfg.hidden_size, self.cfg.ffn_dim, px.Qn
        Hl, Fl = self.h_hi - self.h_lo, self.f_hi - self.f_lo
        hc, fc = H // 256, Fd // 256
        order = [(g + 1 + k) % self.world for k in range(self.world)]   # every rank starts with its successor

        def ln_rows_to_all(x, d, ln):   # x + d, LayerNorm, pack: own tokens -> rows [g*Qn, (g+1)*Qn) of R on every rank
            if self.fuse_ln:
                q8p, scp = px.ptrs("R_q8", g * Qn * H), px.ptrs("R_sc", g * Qn * hc * 4)
                x = ops.add_ln_pack(x, d, ln, [q8p[r] for r in order], H, [scp[r] for r in order], hc)
                px.barrier()
                return x
            if d is not None:
                x = x + d
            px.pack_to_all(ln(x), ops.dp, "R_q8", "R_sc", g * Qn * H, g * Qn * hc * 4, H, hc, Qn)
            return x

        def to_owner(q8, sc, keys, bias):   # [Q, H/G] output block -> column block g of T on each token's owner
            m.linear_from_packed_scatter(q8, sc, keys, bias, ops.dp, dt, False, px.ptrs("T", g * Hl * px.esz), Qn, H)
            px.barrier()

        x_loc = ln_rows_to_all(x_loc, delta, self.self_attn_layer_norm)
        qkv = ops.linear(px.R_q8, px.R_sc, self.keys_qkv, self.bias_qkv, dt)          # [Q, 3 * H/G]
        attn = self._attention(qkv, B, T)
        px.pack_to_all(attn, ops.dp, "C1_q8", "C1_sc", g * Hl, g * (Hl // 256) * 4, H, hc, px.Q)
        to_owner(px.C1_q8, px.C1_sc, self.keys_out, self.bias_out)
        x_loc = ln_rows_to_all(x_loc, px.T, self.final_layer_norm)
        if self.fuse_requant:
            # fc1 -> ReLU -> re-quantise in the fc1 epilogue, stored into C2 of every rank while the dot runs
            q8p, scp = px.ptrs("C2_q8", g * Fl), px.ptrs("C2_sc", g * (Fl // 256) * 4)
            ops.linear_requant(px.R_q8, px.R_sc, self.keys_fc1, self.bias_fc1, dt, True, [q8p[r] for r in order], Fd,
                               [scp[r] for r in order], fc)
            px.barrier()
        else:
            f = ops.linear(px.R_q8, px.R_sc, self.keys_fc1, self.bias_fc1, dt, relu=True)  # [Q, F/G]
            px.pack_to_all(f, ops.dp, "C2_q8", "C2_sc", g * Fl, g * (Fl // 256) * 4, Fd, fc, px.Q)
        to_owner(px.C2_q8, px.C2_sc, self.keys_fc2, self.bias_fc2)
        return x_loc, px.T

    def forward(self, x_loc, delta, B, T, px=None):
        """(x, delta) -> (x, delta): `delta` is the fc2 output of the previous layer for the own tokens, not yet
        added to the residual stream `x` (None at the first layer)."""
        if px is not None:
            return self.forward_peer(x_loc, delta, B, T, px)
        Q = B * T
        ops, dt = self.ops, self.dtype
        H = self.cfg.hidden_size

        def ln_pack(x, d, ln):
            if self.fuse_ln and self.world == 1:
                q8 = torch.empty(Q, H, dtype=torch.int8, device=x.device)
                sc = torch.empty(Q, H // 256, dtype=torch.float32, device=x.device)
                x = ops.add_ln_pack(x, d, ln, [q8.data_ptr()], H, [sc.data_ptr()], H // 256)
                return x, q8, sc
            if d is not None:
                x = x + d
            q8, sc = self._pack_gather_rows(ln(x), Q)
            return x, q8, sc

        x_loc, q8, sc = ln_pack(x_loc, delta, self.self_attn_layer_norm)
        qkv = ops.linear(q8, sc, self.keys_qkv, self.bias_qkv, dt)                   # [Q, 3 * H/G]
        attn = self._attention(qkv, B, T)
        q8, sc = self._pack_gather_cols(attn)
        o = ops.linear(q8, sc, self.keys_out, self.bias_out, dt)                      # [Q, H/G]
        x_loc, q8, sc = ln_pack(x_loc, self._to_token_shard(o), self.final_layer_norm)
        if self.fuse_requant and self.world == 1:
            Fd = self.cfg.ffn_dim
            q8f = torch.empty(Q, Fd, dtype=torch.int8, device=x_loc.device)
            scf = torch.empty(Q, Fd // 256, dtype=torch.float32, device=x_loc.device)
            ops.linear_requant(q8, sc, self.keys_fc1, self.bias_fc1, dt, True, [q8f.data_ptr()], Fd, [scf.data_ptr()], Fd // 256)
            q8, sc = q8f, scf
        else:
            f = ops.linear(q8, sc, self.keys_fc1, self.bias_fc1, dt, relu=True)       # [Q, F/G]
            q8, sc = self._pack_gather_cols(f)
        o = ops.linear(q8, sc, self.keys_fc2, self.bias_fc2, dt)                      # [Q, H/G]
        return x_loc, self._to_token_shard(o)


class TPOPTForCausalLM(nn.Module):
    """OPT with tensor-parallel BSI decoder layers; embeddings, final LayerNorm and lm_head are replicated."""

    def __init__(self, cfg: OPTConfig, rank=0, world=1, group=None, ops=None, dtype=torch.float16, device="cuda",
                 exchange="auto", microbatches=2, fuse_ln=False, peer_timeout_ms=30000, check_status=True):
        super().__init__()
        self.config, self.rank, self.world, self.group, self.dtype = cfg, rank, world, group, dtype
        self.microbatches = int(microbatches)
        self.peer_timeout_ms = int(peer_timeout_ms)
        # After every forward / next_token the device status word is read (this synchronises the device): a bounded
        # wait that gave up (a peer that never arrived: 64 + its rank) or a re-quantised chunk holding inf / NaN (48)
        # raises instead of returning values computed from stale or zeroed buffers. Loops that time the forward set
        # this to False and read the status once at the end.
        self.check_status = bool(check_status)
        self.ops = ops if ops is not None else BsiDeviceOps()
        if exchange not in ("auto", "peer", "collective"):
            raise ValueError("exchange must be auto, peer or collective")
        # peer stores need the CUDA extension; stand-in ops (CPU tests) always use the collectives
        self.exchange = ("peer" if isinstance(self.ops, BsiDeviceOps) else "collective") if exchange == "auto" else exchange
        self._px = {}
        self._streams = None
        H = cfg.hidden_size
        self.embed_tokens = nn.Embedding(cfg.vocab_size, H, padding_idx=1, device=device, dtype=dtype)
        self.embed_positions = nn.Embedding(cfg.max_position_embeddings + 2, H, device=device, dtype=dtype)
        self.final_layer_norm = nn.LayerNorm(H, device=device, dtype=dtype)
        self.layers = nn.ModuleList(
            [TPDecoderLayer(cfg, rank, world, group, self.ops, dtype, device, fuse_ln) for _ in range(cfg.num_hidden_layers)])

    def _stack(self, input_ids, px):
        """Embeddings, decoder layers and final LayerNorm for the rank's own tokens of `input_ids` [b, T]."""
        b, T = input_ids.shape
        Q, G = b * T, self.world
        Qn = Q // G
        ids = input_ids.reshape(Q)[self.rank * Qn:(self.rank + 1) * Qn]
        pos = torch.arange(self.rank * Qn, (self.rank + 1) * Qn, device=input_ids.device) % T + 2   # OPT's offset
        x, delta = self.embed_tokens(ids) + self.embed_positions(pos), None
        for layer in self.layers:
            x, delta = layer(x, delta, b, T, px)
        return self.final_layer_norm(x + delta)

    def _micro(self, B, T):
        """Number of micro-batches for a [B, T] input: with peer exchange the batch is split into groups of
        sequences that run on streams of their own, so that one group's exchange stores and barriers
        overlap the other's kernels."""
        M = self.microbatches if (self.world > 1 and self.exchange == "peer") else 1
        while M > 1 and (B % M != 0 or ((B // M) * T // self.world) % 32 != 0):
            M -= 1
        return max(M, 1)

    @torch.no_grad()
    def _local_hidden(self, input_ids):
        """Final-LayerNorm hidden states of the rank's own tokens: a list with one [Q_m/G, H] tensor per
        micro-batch (micro-batch m holds sequences [m*B/M, (m+1)*B/M))."""
        B, T = input_ids.shape
        G = self.world
        if (B * T) % G != 0:
            raise ValueError("batch x seq must divide evenly over the ranks")
        if not (G > 1 and self.exchange == "peer"):
            return [self._stack(input_ids, None)]
        M = self._micro(B, T)
        b = B // M
        dev = input_ids.device
        pxs = [self._peer_exchange(m, b * T, dev) for m in range(M)]
        if M == 1:
            return [self._stack(input_ids, pxs[0])]
        if self._streams is None or len(self._streams) < M:
            self._streams = [torch.cuda.Stream(dev) for _ in range(M)]
        cur = torch.cuda.current_stream(dev)
        outs = []
        for m in range(M):
            self._streams[m].wait_stream(cur)
        # layer by layer, alternating between the micro-batches, so that the host enqueues them interleaved
        xs, deltas = [], [None] * M
        for m in range(M):
            with torch.cuda.stream(self._streams[m]):
                ids_m = input_ids[m * b:(m + 1) * b]
                Qn = b * T // G
                ids = ids_m.reshape(b * T)[self.rank * Qn:(self.rank + 1) * Qn]
                pos = torch.arange(self.rank * Qn, (self.rank + 1) * Qn, device=dev) % T + 2
                xs.append(self.embed_tokens(ids) + self.embed_positions(pos))
        for layer in self.layers:
            for m in range(M):
                with torch.cuda.stream(self._streams[m]):
                    xs[m], deltas[m] = layer(xs[m], deltas[m], b, T, pxs[m])
        for m in range(M):
            with torch.cuda.stream(self._streams[m]):
                out = self.final_layer_norm(xs[m] + deltas[m])
                out.record_stream(cur)
                outs.append(out)
        for m in range(M):
            cur.wait_stream(self._streams[m])
        return outs

    @torch.no_grad()
    def capture(self, B, T):
        """Records the decoder stack for [B, T] token ids as a CUDA graph; later calls with that shape replay
        it (no per-kernel launch cost on the host). Needs the peer exchange or a single rank: the library
        collectives of the other mode stay outside graphs here. Every rank must call it."""
        if self.world > 1 and self.exchange != "peer":
            raise ValueError("capture needs exchange='peer' when there is more than one rank")
        dev = self.embed_tokens.weight.device
        self._graph = None
        self._g_ids = torch.zeros(B, T, dtype=torch.long, device=dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):      # lazy initialisation (peer buffers, kernel attributes, attention plans)
            for _ in range(2):
                self._local_hidden(self._g_ids)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        if self.world > 1:
            dist.barrier(group=self.group)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._g_out = self._local_hidden(self._g_ids)     # list, one tensor per micro-batch
        self._graph, self._graph_shape = graph, (B, T)
        return self

    @torch.no_grad()
    def hidden_states(self, input_ids):
        """Final-LayerNorm hidden states of all tokens, [B, T, H] (gathered on every rank)."""
        B, T = input_ids.shape
        Q, G = B * T, self.world
        if getattr(self, "_graph", None) is not None and self._graph_shape == (B, T):
            self._g_ids.copy_(input_ids, non_blocking=True)
            self._graph.replay()
            parts = self._g_out
        else:
            parts = self._local_hidden(input_ids)
        if G > 1:
            fulls = []
            for x in parts:      # token shards of one micro-batch -> all of its tokens, in sequence order
                full = torch.empty(x.shape[0] * G, x.shape[1], dtype=x.dtype, device=x.device)
                dist.all_gather_into_tensor(full, x.contiguous(), group=self.group)
                fulls.append(full)
            x = fulls[0] if len(fulls) == 1 else torch.cat(fulls, dim=0)
        else:
            x = parts[0]
        return x.view(B, T, -1)

    def _peer_exchange(self, slot, Q, device):
        """The peer buffers of micro-batch `slot` for Q tokens (built on first use; every rank must get here
        with the same Q)."""
        px = self._px.get(slot)
        if px is not None and px.Q != Q:
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)     # nobody still writes into the buffers about to be unmapped
            px.close()
            px = None
        if px is None:
            if (Q // self.world) % 32 != 0:
                raise ValueError("peer exchange needs a multiple of 32 tokens per rank")
            px = PeerExchange(self.ops.m, self.rank, self.world, self.group, Q, self.config.hidden_size,
                              self.config.ffn_dim, self.dtype, device, timeout_ms=self.peer_timeout_ms)
            self._px[slot] = px
        return px

    def _raise_on_device_status(self):
        if not (self.check_status and isinstance(self.ops, BsiDeviceOps)):
            return
        status = int(self.ops.m.device_status())
        if status == 0:
            return
        if status >= 64:
            what = f"rank {status - 64} never arrived at a peer barrier within {self.peer_timeout_ms} ms"
        elif status == 48:
            what = "a re-quantised chunk held inf, NaN or a value beyond the exact range and was stored as zeros"
        else:
            what = "a bounded wait inside a dot kernel gave up"
        raise RuntimeError(f"BSI device status {status} on rank {self.rank}: {what}; this forward's values are not valid")

    @torch.no_grad()
    def forward(self, input_ids):
        out = F.linear(self.hidden_states(input_ids), self.embed_tokens.weight)
        self._raise_on_device_status()
        return out

    @torch.no_grad()
    def next_token(self, input_ids):
        """Last-position argmax, the reference's accuracy statistic (benchmark_performance_bsi.py:209-212)."""
        tok = F.linear(self.hidden_states(input_ids)[:, -1, :], self.embed_tokens.weight).argmax(dim=-1)
        self._raise_on_device_status()
        return tok


@torch.no_grad()
def build_opt_tp(name="opt-6.7b", dtype=torch.float16, device="cuda", seed=0, decimal_places=2,
                 compress_threshold=0.5, rank=0, world=1, group=None, ops=None, exchange="auto",
                 microbatches=2, fuse_ln=False, peer_timeout_ms=30000, check_status=True):
    """Random-init tensor-parallel OPT. Draws every parameter from the generator `build_opt_bsi` uses for
    it (seeded by the parameter's position in the sorted HF names), so the two models hold the same
    weights, and builds the keys layer by layer so that the dense weights never sit in memory at once."""
    cfg = CONFIGS[name] if isinstance(name, str) else name
    if ops is None:
        ops = BsiDeviceOps(decimal_places, compress_threshold)
    model = TPOPTForCausalLM(cfg, rank, world, group, ops, dtype, device, exchange, microbatches, fuse_ln, peer_timeout_ms,
                             check_status)
    H, Fd, L = cfg.hidden_size, cfg.ffn_dim, cfg.num_hidden_layers
    shapes = {"model.decoder.embed_tokens.weight": (cfg.vocab_size, H),
              "model.decoder.embed_positions.weight": (cfg.max_position_embeddings + 2, H),
              "model.decoder.final_layer_norm.weight": (H,), "model.decoder.final_layer_norm.bias": (H,)}
    lin_shapes = {"q_proj": (H, H), "k_proj": (H, H), "v_proj": (H, H), "out_proj": (H, H), "fc1": (Fd, H), "fc2": (H, Fd)}
    for li in range(L):
        pre = f"model.decoder.layers.{li}."
        for ln in ("self_attn_layer_norm", "final_layer_norm"):
            shapes[pre + ln + ".weight"] = (H,)
            shapes[pre + ln + ".bias"] = (H,)
        for lname, shp in lin_shapes.items():
            owner = pre + ("self_attn." if lname.endswith("proj") else "")
            shapes[owner + lname + ".weight"] = shp
            shapes[owner + lname + ".bias"] = (shp[0],)
    index = {n: i for i, n in enumerate(sorted(shapes))}

    def draw(pname):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + index[pname])
        return torch.empty(shapes[pname], dtype=torch.float32, device=device).normal_(0.0, cfg.init_std, generator=g)

    model.embed_tokens.weight.copy_(draw("model.decoder.embed_tokens.weight").to(dtype))
    model.embed_tokens.weight[1].zero_()
    model.embed_positions.weight.copy_(draw("model.decoder.embed_positions.weight").to(dtype))
    for ln in [model.final_layer_norm] + [m for l in model.layers for m in (l.self_attn_layer_norm, l.final_layer_norm)]:
        ln.weight.fill_(1.0)
        ln.bias.zero_()
    for li, layer in enumerate(model.layers):
        pre = f"model.decoder.layers.{li}."
        weights, biases = {}, {}
        for lname, shp in lin_shapes.items():
            owner = pre + ("self_attn." if lname.endswith("proj") else "")
            weights[lname] = draw(owner + lname + ".weight")
            biases[lname] = torch.zeros(shp[0], dtype=torch.float32, device=device)
        layer.load_linears(weights, biases)
        del weights
    for p in model.parameters():
        p.requires_grad_(False)
    return model.eval()
