"""Decoder-only causal LM shared by the dense and MoE families.

Public surface (reference: minitrain/model/transformer.py:11-161):
``MiniTransformer(cfg, ops, activation_dtype=)``, ``forward(input_ids, targets,
use_fused_loss) -> (loss, logits_or_hidden)``, ``hidden_states(input_ids,
embedding_delta=)``, ``last_training_metrics`` and ``last_training_visualizations``.
"""

from __future__ import annotations

import torch
from torch import nn

from mini_train_sys_b200.models.blocks import RMSNorm, TransformerBlock, project
from mini_train_sys_b200.models.config import ModelConfig
from mini_train_sys_b200.models.ops import OpsBackend
from mini_train_sys_b200.models.rotary import RotaryEmbedding

_ACTIVATION_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


class MiniTransformer(nn.Module):
    def __init__(self, cfg: ModelConfig, ops: OpsBackend, *, activation_dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        if activation_dtype not in _ACTIVATION_DTYPES:
            raise ValueError(f"Unsupported activation dtype: {activation_dtype}")
        self.cfg = cfg
        self.ops = ops
        self.activation_dtype = activation_dtype
        # Construction order fixes the RNG stream and therefore the initial weights.
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.dropout = nn.Dropout(cfg.dropout)
        self.rotary = RotaryEmbedding(cfg.head_dim, cfg.seq_len, cfg.rope_theta, cache_dtype=activation_dtype)
        self.blocks = nn.ModuleList(TransformerBlock(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        nn.init.normal_(self.embed.weight, mean=0.0, std=0.02)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.embed.weight
        else:
            nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.02)
        self.last_training_metrics: dict[str, torch.Tensor] = {}
        self.last_training_visualizations: dict[str, torch.Tensor] = {}
        self._aux: torch.Tensor | None = None
        self._zloss: torch.Tensor | None = None

    # Older experiment code reads these names.
    @property
    def last_moe_metrics(self) -> dict[str, torch.Tensor]:
        return self.last_training_metrics

    @property
    def last_moe_visualizations(self) -> dict[str, torch.Tensor]:
        return self.last_training_visualizations

    def hidden_states(self, input_ids: torch.Tensor, *, embedding_delta: torch.Tensor | None = None) -> torch.Tensor:
        """Final-norm hidden states; never materialises vocabulary logits.

        ``embedding_delta`` is an additive, differentiable perturbation of the token
        embeddings with the same shape; probes train it against a frozen backbone.
        """

        h = None
        own_embedding = getattr(self.ops, "embedding", None)
        if own_embedding is not None and embedding_delta is None and self.activation_dtype == torch.bfloat16:
            h = own_embedding(input_ids, self.embed.weight)      # None when the backend does not cover these inputs
        if h is None:
            h = self.embed(input_ids)
        if embedding_delta is not None:
            if embedding_delta.shape != h.shape:
                raise ValueError("embedding_delta must match embedded input shape")
            h = h + embedding_delta
        h = self.dropout(h.to(self.activation_dtype))
        cos, sin = self.rotary(h.shape[1])
        if cos.device != h.device or cos.dtype != h.dtype:
            raise RuntimeError("RoPE cache must match the residual device and dtype")

        aux, zl = [], []
        per_layer: dict[str, list[torch.Tensor]] = {}
        for block in self.blocks:
            out = block(h, self.ops, cos, sin)
            h = out.hidden_states
            if out.router_aux_loss is not None:
                aux.append(out.router_aux_loss)
            if out.router_z_loss is not None:
                zl.append(out.router_z_loss)
            if out.router_metrics:
                for key, value in out.router_metrics.items():
                    per_layer.setdefault(key, []).append(value)

        scalars: dict[str, torch.Tensor] = {}
        images: dict[str, torch.Tensor] = {}
        for key, values in per_layer.items():
            stack = torch.stack(values)
            if stack.ndim == 1:
                scalars[key] = stack.float().mean()
            else:  # [layer, expert]
                stack = stack.detach()
                images[f"{key}_by_layer"] = stack
                for e, v in enumerate(stack.mean(dim=0)):
                    scalars[f"{key}/expert_{e:02d}"] = v
        self._aux = torch.stack(aux).mean() if aux else None
        self._zloss = torch.stack(zl).mean() if zl else None
        if self._aux is not None:
            scalars["moe/aux_loss"] = self._aux.detach()
        if self._zloss is not None:
            scalars["moe/z_loss"] = self._zloss.detach()
        self.last_training_metrics = scalars
        self.last_training_visualizations = images
        return self.norm(h, self.ops)

    def _lm_loss(self, hidden: torch.Tensor, targets: torch.Tensor, fused: bool) -> tuple[torch.Tensor, torch.Tensor]:
        if fused:
            loss = self.ops.fused_linear_cross_entropy(
                hidden.reshape(-1, hidden.shape[-1]), self.lm_head.weight, targets.reshape(-1))
            return loss, hidden
        logits = project(self.ops, self.lm_head, hidden)
        return self.ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1)), logits

    def forward(self, input_ids: torch.Tensor, targets: torch.Tensor | None = None, use_fused_loss: bool = False
                ) -> tuple[torch.Tensor | None, torch.Tensor]:
        hidden = self.hidden_states(input_ids)
        if targets is None:
            return None, project(self.ops, self.lm_head, hidden)
        lm, out = self._lm_loss(hidden, targets, use_fused_loss)
        m = self.last_training_metrics
        m["loss/lm_cross_entropy"] = lm.detach()
        total = lm
        reg = lm.new_zeros(())
        if self._aux is not None:
            term = self.cfg.router_aux_loss_coef * self._aux
            total, reg = total + term, reg + term
            m["loss/moe_aux_weighted"] = term.detach()
        if self._zloss is not None:
            term = self.cfg.router_z_loss_coef * self._zloss
            total, reg = total + term, reg + term
            m["loss/moe_z_weighted"] = term.detach()
        if self.cfg.is_moe:
            m["loss/moe_regularization_total"] = reg.detach()
        m["loss/total"] = total.detach()
        return total, out


class MiniMoETransformer(MiniTransformer):
    def __init__(self, cfg: ModelConfig, ops: OpsBackend, **kwargs) -> None:
        if not cfg.is_moe:
            raise ValueError("MiniMoETransformer requires ffn_type='moe'")
        super().__init__(cfg, ops, **kwargs)
