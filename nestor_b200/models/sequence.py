"""``SequenceModel(adapter, backbone, head)`` and the ``Model.from_config`` factory.

Parity targets: ``nestor/models/sequence.py:40-179`` (composition, fused head hand-off),
``nestor/adapters/text.py:120-180`` (embedding x ``embedding_multiplier``, trivial-mask
contract: pre-tokenised tensors carry no attention mask), ``nestor/heads/language_modeling.py:85-98``
(``logits = projection(h) * logit_multiplier``).
"""

from __future__ import annotations

import dataclasses as dc
import os
from typing import Any

import torch
from torch import Tensor, nn

from nestor_b200 import ops
from nestor_b200.configs.model import (
    LanguageModelingHeadConfig, NestorConfig, ReferenceMupConfig, SequenceModelConfig, TextAdapterConfig,
)
from nestor_b200.models.modules import LayerStack, Matrix
from nestor_b200.models.nestor import Nestor, W
from nestor_b200.models.registry import (
    ADAPTERS, BACKBONES, HEADS, MODELS, register_adapter, register_backbone, register_head, register_model,
)
from nestor_b200.models.scaling import _ACTIVATIONS as SCALING_ACTIVATIONS, RMSNorm, ScaledLinear
from nestor_b200.models.tags import ADAMW_DECAY, ParamTag, tag


@dc.dataclass
class ModelOutput:
    """``pred``: logits ``[B, S, V]`` — or the head input ``[B, S, d]`` when the head is fused
    into the loss — and ``aux``: routing indices per block plus the fused-head handle."""

    pred: Tensor
    aux: dict[str, Any]


class ByteTokenizer:
    """UTF-8 bytes as token ids (``tokenizer="bytes"``): needs no vocabulary file, for tests and offline use."""

    n_vocab = 256

    def encode_ordinary(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: list[int]) -> str:
        return bytes(int(i) & 0xFF for i in ids).decode("utf-8", errors="replace")


@register_adapter(TextAdapterConfig)
class TextAdapter(nn.Module):
    """Token embedding table; output ``norm(E[ids]) * embedding_multiplier`` in fp32.

    Without a reference-muP recipe the embeddings are normalised to unit RMS (learned gain) before the first block, as
    in the reference's adapter (``nestor/adapters/text.py:71-75,150``); the recipe replaces that norm by the identity
    and scales by its embedding multiplier instead (``nestor/scaling/reference_mup.py:320``).

    The adapter is also the tokenizer for string inputs (reference ``nestor/adapters/text.py:59-101``): a tiktoken
    encoding named by ``config.tokenizer`` (loaded lazily; pre-tokenised tensors never need it), or the built-in
    ``"bytes"`` tokenizer. ``encode_texts`` right-pads a batch to its longest entry (capped at ``max_length``) and
    returns the validity mask; pre-tokenised tensors carry no mask (every position is a real token).
    """

    def __init__(self, config: TextAdapterConfig, mup: ReferenceMupConfig | None) -> None:
        super().__init__()
        if config.vocab_size is None:
            raise ValueError("TextAdapterConfig.vocab_size is required (token ids are the only input form).")
        self.config = config
        self.embed = nn.Embedding(config.vocab_size, config.embed_dim)
        tag(self.embed.weight, ADAMW_DECAY)
        std = mup.initializer_range if mup is not None else 1.0
        nn.init.normal_(self.embed.weight, 0.0, std)
        self.embedding_multiplier = mup.embedding_multiplier if mup is not None else 1.0
        self.norm = RMSNorm(config.embed_dim) if mup is None else None
        self._tokenizer: Any = None

    def tokenizer(self) -> Any:
        if self._tokenizer is None:
            if self.config.tokenizer == "bytes":
                self._tokenizer = ByteTokenizer()
            else:
                try:
                    import tiktoken
                    self._tokenizer = tiktoken.get_encoding(self.config.tokenizer)
                except Exception as exc:   # no package, or no vocabulary file on a machine without network
                    raise RuntimeError(f"cannot load the {self.config.tokenizer!r} tokenizer for string inputs: {exc}. "
                                       "Pass token-id tensors, or use tokenizer='bytes'.") from exc
        return self._tokenizer

    def encode_texts(self, texts: list[str], device: torch.device | None = None) -> tuple[Tensor, Tensor]:
        """``(ids [B, L] int64, valid [B, L] bool)`` for a batch of strings, right-padded with id 0."""

        tok = self.tokenizer()
        rows = [tok.encode_ordinary(t)[: self.config.max_length] for t in texts]
        if any(max(r, default=0) >= self.embed.num_embeddings for r in rows):
            raise ValueError("the tokenizer produced an id beyond the embedding table")
        L = max(1, max(len(r) for r in rows))
        ids = torch.zeros(len(rows), L, dtype=torch.long)
        valid = torch.zeros(len(rows), L, dtype=torch.bool)
        for i, r in enumerate(rows):
            ids[i, : len(r)] = torch.tensor(r, dtype=torch.long)
            valid[i, : len(r)] = True
        device = self.embed.weight.device if device is None else device
        return ids.to(device), valid.to(device)

    def forward(self, ids: Tensor) -> Tensor:
        x = self.embed(ids).float()
        if self.norm is not None:
            x = self.norm(x)
        return x * self.embedding_multiplier


@register_head(LanguageModelingHeadConfig)
class LanguageModelingHead(nn.Module):
    """Unembedding ``[V, d]``, optionally behind hidden layers; ``logit_multiplier = 1 / width_multiplier`` under muP.

    ``hidden_dims`` (usually empty) inserts in-stream layers with ``activation`` between the backbone features and the
    vocabulary matrix (reference ``nestor/heads/language_modeling.py:70-76``). They run as ``pre``; the vocabulary
    matrix stays a single ``[V, d_last]`` weight so that the fused head + cross-entropy kernel path applies to it
    unchanged.
    """

    def __init__(self, config: LanguageModelingHeadConfig, dim: int, mup: ReferenceMupConfig | None) -> None:
        super().__init__()
        dims = [dim, *config.hidden_dims]
        self.hidden = nn.ModuleList(ScaledLinear(a, b, role="in_stream") for a, b in zip(dims[:-1], dims[1:]))
        if config.activation not in SCALING_ACTIVATIONS:
            raise ValueError(f"Unknown head activation {config.activation!r}.")
        self.activation = config.activation
        last = dims[-1]
        std = mup.initializer_range if mup is not None else 1.0 / last
        self.projection = LayerStack([Matrix(last, config.vocab_size, ADAMW_DECAY, std)])
        self.logit_multiplier = 1.0 / mup.width_multiplier if mup is not None else 1.0
        self.vocab_size = config.vocab_size

    @property
    def weight(self) -> Tensor:
        return self.projection.layers[0].weight

    def pre(self, h: Tensor) -> Tensor:
        """The hidden layers in front of the vocabulary matrix (identity for the usual single-matrix head)."""

        act = SCALING_ACTIVATIONS[self.activation]
        for layer in self.hidden:
            h = act(layer(h.to(layer.weight.dtype)))
        return h

    def forward(self, h: Tensor, cd: torch.dtype) -> Tensor:
        return (self.pre(h).to(cd) @ W(self, self.weight).to(cd).t()) * self.logit_multiplier


register_backbone(NestorConfig)(lambda config, mup, **kw: Nestor(config, mup, **kw))


def apply_recipe_variants(model: nn.Module, mup: ReferenceMupConfig) -> None:
    """Optimizer-tag variants of the reference-muP recipe (``nestor/scaling/reference_mup.py:126-311``).

    The models are built with the tags of the Muon pairing (in-stream matrices Muon, single-matrix routers and path
    gates AdamW at the base rate). This pass applies what differs from it:

    * ``matrix_optimizer="adamw"``: attention and expert matrices move to AdamW at ``1 / width_multiplier`` of the base
      rate; routers follow them unless ``NESTOR_MUP_ROUTER_BASE_LR=1`` keeps them at the base rate (the reference
      transform never marks a router); path gates take the matrix rate. The group router's hidden layers stay Muon.
    * ``group_router_lr="base"``: the group router's score / noise read-outs train at the base AdamW rate instead of
      ``score_lr_mul / hidden``.
    * ``NESTOR_MUP_ROUTER_BASE_INIT=1``: single-matrix routers are re-drawn at ``initializer_range`` instead of
      ``initializer_range / sqrt(width_multiplier)``.
    """

    if not mup.enabled("optimizer"):
        return
    muon_matrices = mup.matrix_optimizer == "muon"
    matrix_lr_mul = 1.0 / mup.width_multiplier
    router_lr_mul = 1.0 if muon_matrices or os.environ.get("NESTOR_MUP_ROUTER_BASE_LR", "0") == "1" else matrix_lr_mul
    router_init = os.environ.get("NESTOR_MUP_ROUTER_BASE_INIT", "0") == "1" and mup.enabled("initialization")

    def adamw(p: Tensor, lr_mul: float) -> None:
        tag(p, ParamTag("adamw", lr_mul=lr_mul, weight_decay=True))

    def router(r) -> None:
        w = r.score_mlp.layers[0].weight
        if len(r.score_mlp.layers) == 1:
            adamw(w, router_lr_mul)
            if router_init:
                with torch.no_grad():
                    w.normal_(0.0, mup.initializer_range)

    for block in model.backbone.blocks:
        for layer in block.layers:
            if not muon_matrices:
                for g in layer.attention_groups:
                    for lin in (g.q_proj, g.k_proj, g.v_proj, g.out_proj):
                        adamw(lin.weight, matrix_lr_mul)
                banks = [b for b in (layer.stacked_moe_bank,) if b is not None]
                if layer.expert_pool is not None:
                    banks += [b for b in (layer.expert_pool.stacked_public, layer.expert_pool.stacked_private) if b is not None]
                for bank in banks:
                    for w in bank.matrices():
                        adamw(w, matrix_lr_mul)
                for expert in [*(layer.shared_experts or []), *layer.dense_shared_experts]:
                    for lin in expert.matrices():
                        adamw(lin.weight, matrix_lr_mul)
            if layer.expert_router is not None:
                router(layer.expert_router)
            pool = layer.expert_pool
            if pool is not None:
                for r in ([pool.public_router] if pool.public_router is not None else []) + list(pool.private_routers):
                    router(r)
                if pool.path_gate is not None:
                    adamw(pool.path_gate.weight, router_lr_mul if muon_matrices else matrix_lr_mul)
        if mup.group_router_lr == "base" and block.spec.G > 1:
            for mlp in (block.group_router.score_mlp, block.group_router.noise_mlp):
                if mlp is not None:
                    adamw(mlp.layers[-1].weight, 1.0)


@register_model(SequenceModelConfig)
class SequenceModel(nn.Module):
    """adapter -> backbone -> head, each built from its config through the registries.

    ``fused_head=True`` (the training default) returns the normalised head input as ``pred``
    and exposes the head through ``aux["fused_head_module"]`` so the loss can run the
    chunked head+cross-entropy without materialising ``[T, V]`` logits.
    """

    def __init__(self, config: SequenceModelConfig) -> None:
        super().__init__()
        self.config = config
        mup = config.reference_mup
        if config.adapter_config.embed_dim != config.backbone_config.input_dim:
            raise ValueError("adapter embed_dim must equal backbone input_dim.")
        dense_no_router = os.environ.get("NESTOR_DENSE_NO_ROUTER", "1") == "1"
        self.adapter = ADAPTERS.build(config.adapter_config, mup)
        self.backbone = BACKBONES.build(config.backbone_config, mup, dense_no_router=dense_no_router)
        self.head = HEADS.build(config.head_config, self.backbone.output_dim, mup)
        if mup is not None:
            apply_recipe_variants(self, mup)
        self.fused_head = False
        self.compute_dtype: torch.dtype | None = None
        # NESTOR_FASTPATH_CHECK=1: the first three kernel-path forwards are repeated on the PyTorch statement of the
        # ops with the same routing and the largest difference is printed (reference nestor/backbones/nestor.py:4868-4884)
        self._fastpath_checks = 3 if os.environ.get("NESTOR_FASTPATH_CHECK") == "1" else 0

    def resolve_compute_dtype(self, device: torch.device) -> torch.dtype:
        if self.compute_dtype is not None:
            return self.compute_dtype
        return torch.bfloat16 if device.type == "cuda" else torch.float32

    def forward(self, ids: Tensor | list[str], pos: Tensor | None = None, noises: list | None = None,
                valid: Tensor | None = None) -> ModelOutput:
        """``ids``: token ids ``[B, S]`` or a list of strings (tokenised by the adapter, right-padded).

        ``valid [B, S]`` marks real tokens of right-padded batches. The decoder is causal, so padding after a
        sequence cannot reach any valid position; the mask only has to keep padding out of what is *counted*: it is
        handed on as ``aux["valid_token_mask"]``, which the loss (targets), the router statistics (loss-free
        balancing, auxiliary losses) and the evaluation metrics honour. Padding must follow the real tokens.
        """

        if isinstance(ids, (list, tuple)) and ids and isinstance(ids[0], str):
            ids, valid = self.adapter.encode_texts(list(ids))
        if valid is not None and bool((valid[:, 1:] & ~valid[:, :-1]).any()):
            raise ValueError("valid_token_mask must be a prefix mask (padding only after the real tokens).")
        if valid is not None and not getattr(self.backbone.config, "causal", True) and not bool(valid.all()):
            raise ValueError("a bidirectional (causal=False) model attends to every position of its sequence: "
                             "padded batches are not supported, pass sequences of equal length")
        B, S = ids.shape
        cd = self.resolve_compute_dtype(ids.device)
        x0 = self.adapter(ids).reshape(B * S, -1)
        if valid is not None:
            x0 = x0 * valid.reshape(B * S, 1).to(x0.dtype)
        if ids.is_cuda and cd != torch.bfloat16 and ops.use_kernels(ids):
            # the kernels compute in bf16; a full-precision forward on a GPU is the PyTorch statement of every op
            with ops.oracle_ops():
                h, aux = self.backbone(x0, B, S, cd, pos=pos, noises=noises)
        elif self._fastpath_checks > 0 and ops.use_kernels(ids) and not torch.cuda.is_current_stream_capturing():
            h, aux = self._checked_forward(x0, B, S, cd, pos, noises)
        else:
            h, aux = self.backbone(x0, B, S, cd, pos=pos, noises=noises)
        if valid is not None:
            aux["valid_token_mask"] = valid
            aux["input_ids"] = ids
            flat = valid.reshape(-1)
            for block in aux["blocks"]:          # the routers' own records carry the mask too
                if "group_router" in block:
                    block["group_router"]["valid_token_mask"] = flat
                for layer in block["layers"]:
                    if "expert_router" in layer:
                        layer["expert_router"]["valid_token_mask"] = flat
        if self.fused_head:
            aux["fused_head_module"] = self.head
            return ModelOutput(pred=self.head.pre(h).view(B, S, -1), aux=aux)
        return ModelOutput(pred=self.head(h, cd).view(B, S, -1), aux=aux)

    def _checked_forward(self, x0: Tensor, B: int, S: int, cd: torch.dtype, pos, noises):
        """Kernel-path forward followed by the same forward on the PyTorch ops, with the first pass's routing replayed
        and the same router noise; prints ``[FASTPATH-CHECK] max|kernels - oracle|`` of the head input."""

        self._fastpath_checks -= 1
        if noises is None and self.training:
            noises = [torch.randn(x0.shape[0], b.spec.G, device=x0.device) if b.spec.G > 1 else None
                      for b in self.backbone.blocks]
        tape = ops.RoutingTape()
        ops.set_routing_tape(tape, "record")
        try:
            h, aux = self.backbone(x0, B, S, cd, pos=pos, noises=noises)
            ops.set_routing_tape(tape, "replay")
            with torch.no_grad(), ops.oracle_ops():
                h_ref, _ = self.backbone(x0.detach(), B, S, cd, pos=pos, noises=noises)
        finally:
            ops.set_routing_tape(None)
        diff = (h.detach().float() - h_ref.float()).abs().max().item()
        print(f"[FASTPATH-CHECK] max|kernels - oracle| = {diff:.3e} (head input, {x0.shape[0]} tokens)", flush=True)
        return h, aux

    # ------------------------------------------------------------------ incremental decoding
    def init_kv_cache(self, batch_size: int, max_len: int, device=None, dtype: torch.dtype = torch.float32):
        device = self.head.weight.device if device is None else device
        return self.backbone.init_kv_cache(batch_size, max_len, device, dtype)

    @torch.no_grad()
    def decode_step(self, ids: Tensor, cache, pos: Tensor | None = None) -> Tensor:
        """Logits ``[B, V]`` of the next position given the new tokens ``ids [B]`` (``cache`` is advanced)."""

        B = ids.shape[0]
        if pos is None:
            pos = torch.full((B,), cache.length, dtype=torch.long, device=ids.device)
        cd = torch.float32 if self.compute_dtype is None else self.compute_dtype
        if ids.device.type != "cuda":
            cd = torch.float32
        x0 = self.adapter(ids.reshape(B, 1)).reshape(B, -1)
        h, _ = self.backbone.forward_step(x0, pos, cache, cd)
        return self.head(h, cd).float()

    @torch.no_grad()
    def generate(self, prompt: Tensor, max_new_tokens: int, temperature: float = 0.0,
                 generator: torch.Generator | None = None) -> Tensor:
        """Greedy (``temperature == 0``) or sampled continuation of ``prompt [B, S0]``; returns ``[B, S0 + new]``."""

        was_training = self.training
        self.eval()
        B, S0 = prompt.shape
        cache = self.init_kv_cache(B, S0 + max_new_tokens, prompt.device)
        logits = None
        for t in range(S0):
            logits = self.decode_step(prompt[:, t], cache)
        out = [prompt]
        for _ in range(max_new_tokens):
            if temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits / temperature, dim=-1), 1, generator=generator).squeeze(1)
            else:
                nxt = logits.argmax(dim=-1)
            out.append(nxt.unsqueeze(1))
            logits = self.decode_step(nxt, cache)
        self.train(was_training)
        return torch.cat(out, dim=1)

    def fsdp2_wrap_order(self) -> list[nn.Module]:
        """Sharding units, in gather order: adapter, each block, backbone tail, head, root."""

        return [self.adapter, *self.backbone.blocks, self.backbone, self.head, self]


class Model:
    """Factory namespace: ``Model.from_config(config)`` builds whatever model is registered for the config's type."""

    @staticmethod
    def from_config(config: Any) -> nn.Module:
        return MODELS.build(config)
