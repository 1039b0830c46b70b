"""`Pi0Inference` for B200: weights, static buffers, scratch and one CUDA graph.

Construction uploads the checkpoint, allocates the static buffer plan, runs the pass three
times to populate the scratch pool, freezes the pool and captures vision + prefix encoder +
all decoder steps into a single graph on a side stream. `forward` copies the three inputs into
their static buffers and replays. Public surface and life cycle follow the reference engine
(`.../h100/pi0/engine.py:26-86`).
"""
from __future__ import annotations

import torch

from flash_vla_b200.models.pi0.spec import weight_shapes
from flash_vla_b200.runtime.cuda import ScratchPool

from . import pipeline
from .backends.cuda import wrappers
from .buffers import allocate_static_buffers
from .ops import op_table


class Pi0Inference:
    """One captured Pi0 forward pass.

    `steps` and `layers` shorten the decoder for bisection, as in the reference: on random
    weights a deep run amplifies any difference between two implementations, so parity is read
    on short runs.
    """

    def __init__(self, checkpoint, num_views: int, chunk_size: int, steps: int = 10,
                 layers: int = 18, fused: bool = True, device: str = "cuda", plan=None,
                 capture: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("Pi0Inference needs a CUDA device; the B200 target has no CPU path")
        self.num_views, self.chunk_size = num_views, chunk_size
        self.steps, self.layers, self.fused = steps, layers, fused
        self.ops = op_table(fused, plan=plan)
        self.prompt_len = int(checkpoint["language_embeds"].shape[0])

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
        self.buffers, self.encoder_seq_len = allocate_static_buffers(
            num_views, chunk_size, self.prompt_len, device)

        wrappers.register_bf16_shadow(self.buffers["decoder_x"], self.buffers["decoder_x_bf16"])
        self.pool = ScratchPool()
        self.graph = None
        if capture:
            self._capture()

    def _run(self):
        """One full pass, in place on the static buffers."""
        b = self.buffers
        if self.prompt_len:
            b["encoder_x"][self.num_views * 256:].copy_(self.weights["language_embeds"])
        with wrappers.use_pool(self.pool):
            pipeline.vision_encoder(self.ops, self.weights, b, self.num_views)
            pipeline.transformer_encoder(self.ops, self.weights, b, self.encoder_seq_len)
            pipeline.transformer_decoder(self.ops, self.weights, b, self.encoder_seq_len,
                                         steps=self.steps, layers=self.layers)

    def _capture(self):
        """Warm up (which fills the scratch pool), freeze the pool, capture one pass."""
        for _ in range(3):
            self._run()
        torch.cuda.synchronize()
        self.pool.freeze()
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.graph.capture_begin()
            self._run()
            self.graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

    def set_prompt(self, ids, embedding_table):
        """Replace the prompt: language_embeds[r] = embedding_table[ids[r]] (row gather on the device).

        The prompt length is fixed at construction (it sets the static buffer plan and the captured graph):
        `ids` must hold exactly `prompt_len` token ids. The gather writes into the static tensor the graph
        reads, so the next `forward` uses the new prompt. An extension: the reference takes only
        precomputed `language_embeds` (engine.py:43, :60).
        """
        ids = torch.as_tensor(ids, dtype=torch.int64).reshape(-1)
        if ids.numel() != self.prompt_len:
            raise ValueError(f"set_prompt: {ids.numel()} ids for an engine built with prompt_len={self.prompt_len}")
        if self.prompt_len == 0:
            return
        target = self.weights["language_embeds"]
        table = embedding_table.to(device=target.device, dtype=torch.bfloat16)
        if table.ndim != 2 or table.shape[1] != target.shape[1]:
            raise ValueError(f"set_prompt: embedding table must be (vocab, {target.shape[1]})")
        self.ops.embed_prompt(table.contiguous(), ids.to(target.device), target)

    def __del__(self):
        try:
            wrappers.unregister_bf16_shadow(self.buffers["decoder_x"])
        except Exception:
            pass

    def forward(self, images, state, noise):
        """Copy the inputs into their static buffers, replay, return the denoised chunk.

        The result is the static `diffusion_noise` buffer itself, not a copy: clone it before
        the next call if it must survive.
        """
        b = self.buffers
        b["observation_images_normalized"].copy_(images, non_blocking=True)
        b["observation_state_normalized"].copy_(state, non_blocking=True)
        b["diffusion_noise"].copy_(noise, non_blocking=True)
        if self.graph is None:
            self._run()
        else:
            self.graph.replay()
        return b["diffusion_noise"]
