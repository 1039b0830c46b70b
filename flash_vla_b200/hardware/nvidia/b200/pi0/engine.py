"""`Pi0Inference` for B200: weights, static buffers, scratch and one CUDA graph.

Construction uploads the checkpoint, allocates the static buffer plan, runs the pass three
times to populate the scratch pool, freezes the pool and captures vision + prefix encoder +
all decoder steps into a single graph on a side stream. `forward` copies the three inputs into
their static buffers and replays. Public surface and life cycle follow the reference engine
(`.../h100/pi0/engine.py:26-86`).

`episodes=E > 1` is the throughput profile, a separate execution plan for a batch of E independent
episodes that share the weights:
  * SigLIP and the prefix encoder run ONCE over all episodes' tokens (M = E x S rows): every vision and
    prefix weight (4.8 of the 5.4 GB) is streamed once for the whole batch and the GEMMs have E times
    the tiles to fill the GPU with; only the attention kernels, which mix tokens, run per episode;
  * each episode has its own KV cache; the action-expert decoder also runs ONCE over all episodes' rows
    (M = E x 51): QKV and the gated FFN as one GEMM over all rows, the two residual projections as the
    weight-streaming cluster GEMM once per episode inside one launch, attention for all episodes in one
    launch of the tcgen05 flash kernel (one grid row per episode, each against its own KV cache). At 2
    episodes (or with `batch_decoder=False`) the decoders run as E single-episode decoders on E streams
    instead, which fill each other's idle SMs and are the faster form there.
    Decoder layer L starts as soon as the batched encoder has produced layer L's prefix K/V.
`batch_prefix=False` keeps the older form (E complete single-episode passes on E streams), whose
per-episode results are bit-identical to the single-episode engine; the batched form runs the same
per-row arithmetic but through differently shaped GEMM launches, so it agrees to rounding.
"""
from __future__ import annotations

import torch

from flash_vla_b200.models.pi0.spec import weight_shapes
from flash_vla_b200.runtime.cuda import ScratchPool

from . import pipeline
from .backends.cuda import wrappers
from .buffers import allocate_batched_buffers, allocate_batched_decoder_buffers, allocate_static_buffers
from .ops import op_table


class Pi0Inference:
    """One captured Pi0 forward pass.

    `steps` and `layers` shorten the decoder for bisection, as in the reference: on random
    weights a deep run amplifies any difference between two implementations, so parity is read
    on short runs.
    """

    def __init__(self, checkpoint, num_views: int, chunk_size: int, steps: int = 10,
                 layers: int = 18, fused: bool = True, device: str = "cuda", plan=None,
                 capture: bool = True, episodes: int = 1, overlap: bool = True, embedding_table=None,
                 batch_prefix: bool = True, batch_decoder=None, tuned_plans="default"):
        if not torch.cuda.is_available():
            raise RuntimeError("Pi0Inference needs a CUDA device; the B200 target has no CPU path")
        if episodes < 1:
            raise ValueError("episodes must be >= 1")
        self.num_views, self.chunk_size = num_views, chunk_size
        self.steps, self.layers, self.fused = steps, layers, fused
        self.episodes = episodes
        # overlap: the decoder's first Euler step runs on a second stream, one layer behind the prefix encoder
        # (decoder layer L only needs the prefix K/V of encoder layer L); same kernels, same results
        self.overlap = bool(overlap) and steps >= 1
        self.ops = op_table(fused, plan=plan)
        # measured-best launch plans per GEMM shape (process-wide): "default" = the table shipped next to the
        # sweep harness, if any; a dict or a path = that table; None = leave the library's cost models alone
        from . import autotune
        table = autotune.load_plans() if tuned_plans == "default" else (
            tuned_plans if isinstance(tuned_plans, dict) or tuned_plans is None else autotune.load_plans(tuned_plans))
        self.tuned_plans = autotune.apply_plans(table) if table is not None else 0
        self.prompt_len = int(checkpoint["language_embeds"].shape[0])
        # With an embedding table the prompt lookup is part of the captured pass: the graph gathers
        # table[prompt_ids] straight into the prefix rows, and `set_prompt(ids)` only rewrites the ids.
        self.embedding_table = None
        self.prompt_ids = None
        if embedding_table is not None and self.prompt_len:
            table = embedding_table.to(device=device, dtype=torch.bfloat16).contiguous()
            if table.ndim != 2 or table.shape[1] != checkpoint["language_embeds"].shape[1]:
                raise ValueError(f"embedding_table must be (vocab, {checkpoint['language_embeds'].shape[1]})")
            self.embedding_table = table
            self.prompt_ids = torch.zeros(self.prompt_len, dtype=torch.int64, device=device)

        expected = weight_shapes(self.prompt_len)
        missing = sorted(set(expected) - set(checkpoint))
        if missing:
            raise KeyError(f"checkpoint is missing tensors: {missing}")
        self.weights = {}
        for name, shape in expected.items():
            value = checkpoint[name]
            if tuple(value.shape) != tuple(shape):
                raise ValueError(f"checkpoint[{name!r}] has shape {tuple(value.shape)}, expected {shape}")
            self.weights[name] = value.to(device=device, dtype=torch.bfloat16).contiguous()
        self.episode_buffers, self.pools = [], []
        self.batch_prefix = bool(batch_prefix) and episodes > 1
        # measured on B200: the batched decoder beats concurrent single-episode decoders from 3 episodes on
        # (E = 3: 11.2 against 13.0 ms, E = 4: 11.7 against 17.4 ms) and loses at 2 (11.5 against 9.1 ms)
        if batch_decoder is None:
            batch_decoder = episodes >= 3
        self.batch_decoder = self.batch_prefix and bool(batch_decoder)
        self.prefix_buffers, self.prefix_pool, self.decoder_buffers = None, None, None
        if self.batch_prefix:
            self.prefix_buffers, self.episode_buffers, self.encoder_seq_len = allocate_batched_buffers(
                num_views, chunk_size, self.prompt_len, episodes, device)
            self.prefix_pool = ScratchPool()
        if self.batch_decoder:
            self.decoder_buffers = allocate_batched_decoder_buffers(chunk_size, episodes, self.encoder_seq_len, device)
            self.decoder_pool = ScratchPool()
            self.pools = [self.decoder_pool]
            self._batched_observation_state_normalized = self.decoder_buffers["observation_state_normalized"]
            self._batched_diffusion_noise = self.decoder_buffers["diffusion_noise"]
            self._batched_observation_images_normalized = self.prefix_buffers["observation_images_normalized"].view(
                episodes, num_views, 224, 224, 3)
            self.streams = [torch.cuda.Stream(device=device)]
        elif self.batch_prefix:
            for buffers in self.episode_buffers:
                wrappers.register_bf16_shadow(buffers["decoder_x"], buffers["decoder_x_bf16"])
                self.pools.append(ScratchPool())
            for name in ("observation_state_normalized", "diffusion_noise"):
                batched = torch.zeros((episodes,) + tuple(self.episode_buffers[0][name].shape), dtype=torch.bfloat16, device=device)
                for e, b in enumerate(self.episode_buffers):
                    b[name] = batched[e]
                setattr(self, "_batched_" + name, batched)
            self._batched_observation_images_normalized = self.prefix_buffers["observation_images_normalized"].view(
                episodes, num_views, 224, 224, 3)
            self.streams = [torch.cuda.Stream(device=device) for _ in range(episodes)]
        else:
            for _ in range(episodes):
                buffers, self.encoder_seq_len = allocate_static_buffers(num_views, chunk_size, self.prompt_len, device)
                wrappers.register_bf16_shadow(buffers["decoder_x"], buffers["decoder_x_bf16"])
                self.episode_buffers.append(buffers)
                self.pools.append(ScratchPool())
        if episodes > 1 and not self.batch_prefix:
            # inputs and the result of all episodes live in three batched tensors, so `forward` stays three copies
            for name in ("observation_images_normalized", "observation_state_normalized", "diffusion_noise"):
                batched = torch.zeros((episodes,) + tuple(self.episode_buffers[0][name].shape), dtype=torch.bfloat16, device=device)
                for e, b in enumerate(self.episode_buffers):
                    b[name] = batched[e]
                setattr(self, "_batched_" + name, batched)
            self.streams = [torch.cuda.Stream(device=device) for _ in range(episodes)]
        self.decoder_streams = [torch.cuda.Stream(device=device) for _ in range(episodes)] if self.overlap and not self.batch_prefix else []
        self.buffers, self.pool = self.episode_buffers[0], self.pools[0]
        self.graph = None
        if capture:
            self._capture()

    def _run_episode(self, e: int):
        b = self.episode_buffers[e]
        if self.prompt_len and self.embedding_table is not None:
            self.ops.embed_prompt(self.embedding_table, self.prompt_ids, b["encoder_x"][self.num_views * 256:])
        elif self.prompt_len:
            b["encoder_x"][self.num_views * 256:].copy_(self.weights["language_embeds"])
        with wrappers.use_pool(self.pools[e]):
            pipeline.vision_encoder(self.ops, self.weights, b, self.num_views)
            if not self.overlap:
                pipeline.transformer_encoder(self.ops, self.weights, b, self.encoder_seq_len)
                pipeline.transformer_decoder(self.ops, self.weights, b, self.encoder_seq_len,
                                             steps=self.steps, layers=self.layers)
                return
            main, side = torch.cuda.current_stream(), self.decoder_streams[e]
            kv_ready = [torch.cuda.Event() for _ in range(pipeline.ENCODER_LAYERS)]
            side.wait_stream(main)
            with torch.cuda.stream(side):
                pipeline.decoder_prologue(self.ops, self.weights, b)
            pipeline.transformer_encoder(self.ops, self.weights, b, self.encoder_seq_len,
                                         after_qkv=lambda layer: kv_ready[layer].record(main))
            with torch.cuda.stream(side):
                pipeline.decoder_step(self.ops, self.weights, b, self.encoder_seq_len, 0, self.layers,
                                      noise=b.get("diffusion_noise_f32"),
                                      before_layer=lambda layer: side.wait_event(kv_ready[layer]))
            main.wait_stream(side)
            pipeline.transformer_decoder(self.ops, self.weights, b, self.encoder_seq_len,
                                         steps=self.steps, layers=self.layers, first_step=1)

    def _run_fully_batched(self):
        """Throughput plan with the decoder batched as well: prefix pass on the current stream, the one
        batched decoder on a second stream, its first step one layer behind the encoder."""
        E, S, p, d = self.episodes, self.encoder_seq_len, self.prefix_buffers, self.decoder_buffers
        main, side = torch.cuda.current_stream(), self.streams[0]
        self._write_prompt_rows()
        side.wait_stream(main)
        with torch.cuda.stream(side), wrappers.use_pool(self.decoder_pool):
            pipeline.decoder_prologue_batched(self.ops, self.weights, d)
        kv_ready = [torch.cuda.Event() for _ in range(pipeline.ENCODER_LAYERS)]
        with wrappers.use_pool(self.prefix_pool):
            pipeline.vision_encoder(self.ops, self.weights, p, self.num_views)
            pipeline.transformer_encoder_batched(self.ops, self.weights, p, S, self.num_views, E,
                                                 after_qkv=lambda layer: kv_ready[layer].record(main),
                                                 per_episode=self._attention_fork())
        with torch.cuda.stream(side), wrappers.use_pool(self.decoder_pool):
            if self.steps == 0:
                side.wait_event(kv_ready[-1])
            for step in range(self.steps):
                gate = (lambda layer: side.wait_event(kv_ready[layer])) if step == 0 else None
                pipeline.decoder_step_batched(self.ops, self.weights, p, d, S, step, E, self.layers, before_layer=gate)
            pipeline.decoder_epilogue_batched(d)
        main.wait_stream(side)

    def _attention_fork(self):
        """`per_episode` hook of the batched prefix encoder: episode e's attention goes to a stream of its own,
        forked from the current stream; the call with None joins them all back."""
        import contextlib
        import os
        if "mma" in (os.environ.get("FVLA_ATTN"), os.environ.get("FVLA_GEMM")):
            return None      # the warp-level fallback shares one split-K scratch between the episodes: keep it serial
        main = torch.cuda.current_stream()
        if not hasattr(self, "_attn_streams"):
            self._attn_streams = [torch.cuda.Stream(device=main.device) for _ in range(self.episodes)]
        used = []

        @contextlib.contextmanager
        def on_stream(e):
            stream = self._attn_streams[e]
            stream.wait_stream(main)
            used.append(stream)
            with torch.cuda.stream(stream):
                yield

        def hook(e):
            if e is None:
                for stream in used:
                    main.wait_stream(stream)
                used.clear()
                return None
            return on_stream(e)
        return hook

    def _write_prompt_rows(self):
        E, S, p = self.episodes, self.encoder_seq_len, self.prefix_buffers
        if not self.prompt_len:
            return
        for e in range(E):
            rows = p["encoder_x"][e * S + self.num_views * 256:(e + 1) * S]
            if self.embedding_table is not None:
                self.ops.embed_prompt(self.embedding_table, self.prompt_ids, rows)
            else:
                rows.copy_(self.weights["language_embeds"])

    def _run_batched(self):
        """The throughput plan: one SigLIP + prefix-encoder pass over all episodes' rows on the current stream,
        the episodes' decoders on one stream each, every decoder layer gated on the batched encoder's K/V."""
        if self.batch_decoder:
            self._run_fully_batched()
            return
        E, S, p = self.episodes, self.encoder_seq_len, self.prefix_buffers
        main = torch.cuda.current_stream()
        self._write_prompt_rows()
        for e, stream in enumerate(self.streams):               # what the decoders can do before any K/V exists
            stream.wait_stream(main)
            with torch.cuda.stream(stream), wrappers.use_pool(self.pools[e]):
                pipeline.decoder_prologue(self.ops, self.weights, self.episode_buffers[e])
        kv_ready = [torch.cuda.Event() for _ in range(pipeline.ENCODER_LAYERS)]
        with wrappers.use_pool(self.prefix_pool):
            pipeline.vision_encoder(self.ops, self.weights, p, self.num_views)
            pipeline.transformer_encoder_batched(self.ops, self.weights, p, S, self.num_views, E,
                                                 after_qkv=lambda layer: kv_ready[layer].record(main),
                                                 per_episode=self._attention_fork())
        for e, stream in enumerate(self.streams):
            b = self.episode_buffers[e]
            with torch.cuda.stream(stream), wrappers.use_pool(self.pools[e]):
                if self.steps >= 1:
                    pipeline.decoder_step(self.ops, self.weights, b, S, 0, self.layers, noise=b.get("diffusion_noise_f32"),
                                          before_layer=lambda layer, st=stream: st.wait_event(kv_ready[layer]))
                else:
                    stream.wait_event(kv_ready[-1])
                pipeline.transformer_decoder(self.ops, self.weights, b, S, steps=self.steps, layers=self.layers,
                                             first_step=min(1, self.steps))
        for stream in self.streams:
            main.wait_stream(stream)

    def _run(self):
        """One full pass per episode, in place on the static buffers; episodes run on streams of their own."""
        if self.batch_prefix:
            self._run_batched()
            return
        if self.episodes == 1:
            self._run_episode(0)
            return
        current = torch.cuda.current_stream()
        for e, stream in enumerate(self.streams):
            stream.wait_stream(current)
            with torch.cuda.stream(stream):
                self._run_episode(e)
        for stream in self.streams:
            current.wait_stream(stream)

    def _capture(self):
        """Warm up (which fills the scratch pool), freeze the pool, capture one pass."""
        for _ in range(3):
            self._run()
        torch.cuda.synchronize()
        for pool in self.pools + ([self.prefix_pool] if self.prefix_pool is not None else []):
            pool.freeze()
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.graph.capture_begin()
            self._run()
            self.graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

    def set_prompt(self, ids, embedding_table=None):
        """Replace the prompt: the prefix rows after the image tokens become embedding_table[ids].

        The prompt length is fixed at construction (it sets the static buffer plan and the captured graph):
        `ids` must hold exactly `prompt_len` token ids. An engine built with `embedding_table=` gathers
        inside its captured pass from a static id buffer; this call then only copies the ids there (a
        table passed here must be omitted). Otherwise the gather runs here, outside the graph, into the
        static `language_embeds` tensor the graph reads. Either way the next `forward` uses the new
        prompt. An extension: the reference takes only precomputed `language_embeds` (engine.py:43, :60).
        """
        ids = torch.as_tensor(ids, dtype=torch.int64).reshape(-1)
        if ids.numel() != self.prompt_len:
            raise ValueError(f"set_prompt: {ids.numel()} ids for an engine built with prompt_len={self.prompt_len}")
        if self.prompt_len == 0:
            return
        if self.embedding_table is not None:
            if embedding_table is not None:
                raise ValueError("set_prompt: this engine gathers from the table given at construction")
            self.prompt_ids.copy_(ids, non_blocking=True)
            return
        if embedding_table is None:
            raise ValueError("set_prompt: an embedding table is needed (none was given at construction)")
        target = self.weights["language_embeds"]
        table = embedding_table.to(device=target.device, dtype=torch.bfloat16)
        if table.ndim != 2 or table.shape[1] != target.shape[1]:
            raise ValueError(f"set_prompt: embedding table must be (vocab, {target.shape[1]})")
        self.ops.embed_prompt(table.contiguous(), ids.to(target.device), target)

    def forward(self, images, state, noise):
        """Copy the inputs into their static buffers, replay, return the denoised chunk.

        The result is the static `diffusion_noise` buffer itself, not a copy: clone it before
        the next call if it must survive. With `episodes=E > 1` the three inputs carry a leading
        dimension E and the result is `(E, chunk, 32)`.
        """
        if self.episodes == 1:
            b = self.buffers
            dst = (b["observation_images_normalized"], b["observation_state_normalized"], b["diffusion_noise"])
        else:
            dst = (self._batched_observation_images_normalized, self._batched_observation_state_normalized,
                   self._batched_diffusion_noise)
        for name, src, to in zip(("images", "state", "noise"), (images, state, noise), dst):
            if tuple(src.shape) != tuple(to.shape):          # copy_ would broadcast silently
                raise ValueError(f"forward: {name} has shape {tuple(src.shape)}, expected {tuple(to.shape)}")
        dst[0].copy_(images, non_blocking=True)
        dst[1].copy_(state, non_blocking=True)
        dst[2].copy_(noise, non_blocking=True)
        if self.graph is None:
            self._run()
        else:
            self.graph.replay()
        return dst[2]
