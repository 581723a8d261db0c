"""One quantized denoising step of the H3-shaped transformer: token embedding, n_blocks fused blocks
(rapid_h3_b200.nodes.FusedBlock), final norm + projection. This is the call a user of the package
makes per sampler step; with `torch.distributed` initialised it runs sequence-parallel (token shards,
Ulysses exchange around self-attention).

Reference: the per-step entry of the node pack is the DIFFUSION_MODEL wrapper that swaps every block's
forward for the fused one (custom_nodes/rapid_h3/__init__.py:398-415); 48-50 blocks x CFG batch per step
(csrc/attn_cake/DESIGN.md:19-22).
"""
import torch

from . import model as M
from . import nodes
from .sp import Ulysses, shard_segments


class H3Runtime:
    """Quantized weights and fused forwards of an H3Transformer, ready to step."""

    def __init__(self, model, mode="int8_rowwise", release_bf16=False):
        self.model = model
        self.cfg = model.cfg
        patched, = nodes.RapidH3LinearQuant().patch(model, mode)
        self.linears, self.blocks = patched.linears, patched.block_forward
        for q in self.linears.values():
            q.qweight_for()
        for fb in self.blocks:
            fb._fc1_swiglu_weight()
        if release_bf16:  # keep only the int8 copies (the 48-block model holds ~16 GB of them)
            for q in self.linears.values():
                q.module.weight.data = torch.empty(0, device=q.module.weight.device, dtype=torch.bfloat16)

    @staticmethod
    def random(cfg, seed, device="cuda", release_bf16=True, mode="int8_rowwise"):
        """Random-init model of the benchmark configurations, generated and quantized block by block on `device`."""
        with torch.device("meta"):
            model = M.H3Transformer(cfg)
        model.to_empty(device=device)
        g = torch.Generator(device=device).manual_seed(seed)
        rt = H3Runtime.__new__(H3Runtime)
        rt.model, rt.cfg = model, cfg
        M.init_weights_on_device(model, g, skip_prefix="blocks.")
        linears, forwards = {}, []
        for i, blk in enumerate(model.blocks):
            M.init_weights_on_device(blk, g)
            qs = {}
            for name in ("attn.qkv_proj", "attn.out_proj", "mlp.fc1", "mlp.fc2", "cross.q_proj", "cross.kv_proj",
                         "cross.out_proj"):
                if name.startswith("cross") and not cfg.cross_attention:
                    continue
                mod = blk.get_submodule(name)
                q = nodes._QuantLinear(mod, f"blocks.{i}.{name}", mode=mode)
                q.qweight_for()
                if release_bf16:
                    mod.weight.data = torch.empty(0, device=device, dtype=torch.bfloat16)
                qs[name] = q
                linears[q.name] = q
            fb = nodes._fused_block(blk, qs["attn.qkv_proj"], qs["attn.out_proj"], qs["mlp.fc1"], qs["mlp.fc2"],
                                    qs.get("cross.q_proj"), qs.get("cross.kv_proj"), qs.get("cross.out_proj"))
            fb._fc1_swiglu_weight()
            forwards.append(fb)
        rt.linears, rt.blocks = linears, forwards
        return rt

    # -------------------------------------------------------------------------------------------
    def step(self, latent, audio, t_emb, rope_freqs, ctx, sp=None, streams=None):
        """One transformer evaluation.

        latent [B, C, T, H, W], audio [B, A, C] (A may be 0), t_emb [B, R, d] (row 0 video, row 1 audio),
        rope_freqs bf16 [S, 48, 2, 2] for the S = T*H*W + A packed tokens, ctx [B, Ttext, text_dim].
        Returns (video [B, C, T, H, W], audio [B, A, C]) in bf16. With `sp` (an Ulysses group over S tokens, or a
        list with one group per sample) every rank passes the same full inputs, computes its token shard and
        receives the full result.

        `streams` (a list of CUDA streams, one per sample) runs the samples of the batch side by side: the samples
        are independent, so while one of them sits in an exchange of the sequence-parallel step (a kernel that only
        stores over NVLink, then a barrier across the ranks) the other one's GEMMs and attention keep the SMs busy.
        Each concurrent sample then needs its own Ulysses group, because a group owns one set of exchange buffers."""
        b = latent.shape[0]
        n_video = latent.shape[2] * latent.shape[3] * latent.shape[4]
        n_audio = audio.shape[1] if audio is not None else 0
        s = n_video + n_audio
        segs = [(0, n_video, 0)] + ([(n_video, s, 1)] if n_audio else [])
        sps = list(sp) if isinstance(sp, (list, tuple)) else [sp] * b
        if len(sps) != b:
            raise RuntimeError(f"{len(sps)} sequence-parallel groups for a batch of {b}")
        if streams is not None:
            if len(streams) != b:
                raise RuntimeError(f"{len(streams)} streams for a batch of {b}")
            if sps[0] is not None and len({id(g) for g in sps}) != b:
                raise RuntimeError("samples that run side by side need one Ulysses group each")
        lo, hi = (0, s) if sps[0] is None else (sps[0].lo, sps[0].hi)
        segs_l = segs if sps[0] is None else shard_segments(segs, lo, hi)
        rope_l = rope_freqs.reshape(s, 48, 2, 2)[lo:hi].contiguous()
        m = self.model
        xs = []
        for i in range(b):
            x = m.tokens(latent[i], None if audio is None else audio[i])  # per-token: embed, then take the shard
            xs.append(x[lo:hi].contiguous())
        if streams is None:
            for fb in self.blocks:        # blocks outermost: a block's weights serve every sample of the batch
                for i in range(b):
                    xs[i] = fb.forward(xs[i], t_emb[i], segs_l, rope_l, ctx[i], sp=sps[i])
        else:
            # what the blocks cache per shape (row index, constant tables) is made here, on the caller's stream,
            # so that no side stream ever reads a cached tensor another side stream is still filling
            nodes.prewarm_constants(self.blocks, hi - lo, segs_l, xs[0].device)
            main = torch.cuda.current_stream()
            for st in streams:
                st.wait_stream(main)
            for fb in self.blocks:
                for i in range(b):
                    with torch.cuda.stream(streams[i]):
                        xs[i] = fb.forward(xs[i], t_emb[i], segs_l, rope_l, ctx[i], sp=sps[i])
            for i, st in enumerate(streams):
                xs[i].record_stream(st)
                main.wait_stream(st)
        vids, auds = [], []
        for i in range(b):
            x = xs[i] if sps[i] is None else sps[i].gather_tokens(xs[i])
            v, a = m.untokens(x, latent.shape[1:])
            vids.append(v), auds.append(a)
        return torch.stack(vids), torch.stack(auds)


def rope_table_for_grid(t, h, w, n_audio=0):
    """bf16 [S, 48, 2, 2] rotation table (cos, -sin, sin, cos) of a T x H x W token grid followed by
    n_audio tokens that advance along t only; 3 axes x 16 frequencies (rot_dim 96, split-half layout)."""
    tt, hh, ww = torch.meshgrid(torch.arange(t), torch.arange(h), torch.arange(w), indexing="ij")
    pos = torch.stack([tt.reshape(-1), hh.reshape(-1), ww.reshape(-1)], 1).double()
    if n_audio:
        a = torch.zeros(n_audio, 3, dtype=torch.float64)
        a[:, 0] = torch.arange(n_audio, dtype=torch.float64) * (t / max(n_audio, 1))
        pos = torch.cat([pos, a], 0)
    pos = pos.to(torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(16, dtype=torch.float32) / 16))
    half = torch.cat((pos.unsqueeze(-1) * inv.view(1, 1, -1)).unbind(1), -1)
    c, s = torch.cos(half), torch.sin(half)
    return torch.stack([c, -s, s, c], -1).reshape(pos.shape[0], 48, 2, 2).to(torch.bfloat16)


def make_inputs(cfg, grid, n_audio, batch, text_len, seed=0):
    """Seeded synthetic step inputs on the CPU: latent ~ N(0,1) on the (T, H, W) token grid, audio tokens,
    a random timestep embedding per modality, text tokens ~ N(0,1), and the rope table of the grid."""
    g = torch.Generator().manual_seed(seed)
    t, h, w = grid
    latent = torch.randn(batch, cfg.latent_ch, t, h, w, generator=g).to(torch.bfloat16)
    audio = torch.randn(batch, n_audio, cfg.latent_ch, generator=g).to(torch.bfloat16)
    t_emb = torch.randn(batch, 2, cfg.d_model, generator=g).to(torch.bfloat16)
    ctx = torch.randn(batch, text_len, cfg.text_dim, generator=g).to(torch.bfloat16)
    return latent, audio, t_emb, rope_table_for_grid(t, h, w, n_audio), ctx
