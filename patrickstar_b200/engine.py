"""``initialize_engine`` — the reference's config surface for the optimizer step.

Mirror of ``patrickstar/runtime/__init__.py:40-93`` and of the configuration
half of ``PatrickStarEngine.__init__`` (``patrickstar/runtime/engine.py:53-126``):
the same nested dict, keys, defaults and quirks.  The forward/backward wrappers
of the reference engine (hooks, memory tracer, chunk eviction) serve model
execution and are not rebuilt; ``ChunkStepEngine`` keeps only a thin
forward / backward / step so that a small model can be trained end to end.

Quirks kept on purpose (they decide the loss-scale trajectory):
  * ``fp16.hysteresis`` is passed as the scaler's ``scale_factor`` and
    ``delayed_shift`` stays 1 (engine.py:90-97): every overflow divides the
    scale by ``hysteresis`` at once.
  * ``fp16`` present requires ``enabled`` true and a ``loss_scale`` key
    (engine.py:84-88); ``loss_scale == 0`` selects the dynamic scaler.
  * ``config=None`` crashes in the reference (``None.get``,
    runtime/__init__.py:74); here it means "all defaults".

One key is added under the reference's ``client.opts`` block
(runtime/__init__.py:60-71 holds ``with_mem_saving_comm`` etc. there):
``fused_collectives`` — how a data-parallel step exchanges chunks.
``"nccl"``: NCCL reduce-scatter / all-gather pipelined around the step kernel,
each group's reduce-scatter fired from the backward hand-off;
``"multimem"`` / ``"p2p"``: one kernel that does the reduction, the step and
the gather over NVSwitch multicast memory or peer mappings; ``"staged"`` /
``"copy"``: the pipelined two-kernel and copy-engine forms of the same exchange;
``"auto"`` (default): p2p for 2-3 ranks, multimem for more, nccl when symmetric
memory cannot be set up.
"""
import torch

from .chunk_list import DEFAULT_CHUNK_SIZE
from .client import ChunkClient
from .fp16_adam import FP16Adam
from .loss_scaler import DynamicLossScaler, LossScaler

_DEFAULT_OPTIM = {
    "type": "Adam",
    "params": {"lr": 0.01, "betas": (0.9, 0.999), "eps": 1e-8, "weight_decay": 0, "use_hybrid_adam": True},
}


def parse_config(config):
    """engine.py:53-105 as a pure function.  Returns a dict with optim_type,
    optim_params, scaler ("none" | ("static", scale) | ("dynamic", kwargs)),
    gradient_clipping, default_chunk_size."""
    out = {"default_chunk_size": DEFAULT_CHUNK_SIZE, "gradient_clipping": -1, "scaler": "none",
           "fused_collectives": "auto"}
    if config is None:
        out["optim_type"] = _DEFAULT_OPTIM["type"]
        out["optim_params"] = dict(_DEFAULT_OPTIM["params"])
        return out
    out["default_chunk_size"] = config.get("default_chunk_size", DEFAULT_CHUNK_SIZE)
    optim_config = config.get("optimizer", _DEFAULT_OPTIM)
    optim_type = optim_config.get("type", _DEFAULT_OPTIM["type"])
    if optim_type not in ["Adam", "AdamW"]:
        raise ValueError(
            f"Only support Adam and AdamW at the moment. Get optimizer type {optim_type}")
    optim_params = dict(optim_config.get("params", _DEFAULT_OPTIM["params"]))
    for key, val in _DEFAULT_OPTIM["params"].items():
        if key not in optim_params:
            optim_params[key] = val
    out["optim_type"] = optim_type
    out["optim_params"] = optim_params
    if "fp16" in config:
        ls = config["fp16"]
        assert ls["enabled"], "Must enable fp16 training."
        assert "loss_scale" in ls, "Must have `loss_scale` field set."
        if ls["loss_scale"] == 0:
            out["scaler"] = ("dynamic", dict(
                init_scale=2 ** ls.get("initial_scale_power", 16),
                scale_factor=ls.get("hysteresis", 2),
                scale_window=ls.get("loss_scale_window", 2000),
                min_scale=ls.get("min_loss_scale", 1)))
        else:
            out["scaler"] = ("static", ls["loss_scale"])
    if "gradient_clipping" in config:
        out["gradient_clipping"] = config["gradient_clipping"]
    mode = ((config.get("client") or {}).get("opts") or {}).get("fused_collectives", "auto")
    if mode not in ("auto", "nccl", "multimem", "p2p", "staged", "copy"):
        raise ValueError("client.opts.fused_collectives must be auto, nccl, multimem, p2p, staged or copy; "
                         "got %r" % (mode,))
    out["fused_collectives"] = mode
    return out


_SYMMETRIC_FORMS = ("multimem", "p2p", "staged", "copy")   # need the fp16 chunk list in symmetric memory


def resolve_collectives(mode, world_size):
    """The transport ``auto`` stands for at a world size."""
    if world_size <= 1:
        return "none"
    if mode == "auto":
        return "p2p" if world_size <= 3 else "multimem"
    return mode


def build_loss_scaler(parsed, device=None):
    s = parsed["scaler"]
    if s == "none":
        return None
    if s[0] == "dynamic":
        return DynamicLossScaler(device=device, **s[1])
    return LossScaler(s[1], device=device)


class ChunkStepEngine(torch.nn.Module):
    """Thin stand-in for PatrickStarEngine: holds module, client, loss scaler and
    optimizer; ``backward`` scales the loss and hands the gradients to the fp16
    slots the way the reference's backward hook does
    (patrickstar/core/hook.py:200-230)."""

    def __init__(self, model, client, config, collectives=None):
        super().__init__()
        self.module = model
        self.client = client
        parsed = parse_config(config)
        self.loss_scaler = build_loss_scaler(parsed, client.device)
        self.gradient_clipping = parsed["gradient_clipping"]
        op = parsed["optim_params"]
        self.optimizer = FP16Adam(
            client, self.module.parameters(), loss_scaler=self.loss_scaler,
            gradient_clipping=self.gradient_clipping, lr=op["lr"], betas=op["betas"], eps=op["eps"],
            weight_decay=op["weight_decay"], use_adamw=(parsed["optim_type"] == "AdamW"),
            use_hybrid_adam=op["use_hybrid_adam"])
        # how a data-parallel step exchanges chunks; the fused forms need the fp16 chunk list
        # in symmetric memory
        want = collectives or resolve_collectives(parsed["fused_collectives"], client.world_size)
        if want in _SYMMETRIC_FORMS and client.symm_handle is None:
            want = "nccl"
        self.collectives = want
        # NCCL form: a group's reduce-scatter starts as soon as its gradients are complete
        self.optimizer.rs_on_handoff = (want == "nccl")
        # hand every chunk-managed gradient off the moment autograd has accumulated it, so
        # that the overflow test, the copy into the slot and the reduce-scatter trigger run
        # inside backward (patrickstar/core/hook.py:205-230)
        self._hooks = []
        for p in self.module.parameters():
            if p.requires_grad and p.dtype == torch.float16:
                self._hooks.append(p.register_post_accumulate_grad_hook(self.optimizer.handoff_grad))

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def backward(self, loss):
        """engine.py:206-224 + hook.py:212-216: scaled backward, per-parameter
        overflow check, gradient copied into the parameter's fp16 slot."""
        if self.loss_scaler is not None:
            self.loss_scaler.backward(loss)
        else:
            loss.backward()
        for p in self.module.parameters():
            self.optimizer.handoff_grad(p)   # whatever the hooks did not see (no-op otherwise)
        self._grads_scanned = True

    def step(self):
        """optimizer.step() without a second overflow scan when every gradient came
        through ``backward`` above."""
        scanned, self._grads_scanned = getattr(self, "_grads_scanned", False), False
        if self.client._budget == "auto":
            # hybrid placement follows the memory that is free now, step by step
            # (patrickstar/ops/fp16_cpu_adam.py:523-528); moves nothing while the split holds
            self.optimizer.rebalance()
        if self.client.world_size > 1:
            # data parallel: reduce-scatter of the gradient chunks, rank-local step,
            # all-gather of the param chunks (patrickstar/core/client.py:818-856, 428-497)
            # (chunks whose state lives in pinned host memory go through the offload pipeline,
            # which the NCCL form drives; it works on symmetric memory as well)
            if self.collectives in _SYMMETRIC_FORMS and self.optimizer._offload is None:
                return self.optimizer.step_fused_collectives(self.collectives, scan="done" if scanned else "local")
            return self.optimizer.step_with_collectives(scan="done" if scanned else "local")
        return self.optimizer.step(scan=not scanned)


def _client_for(parsed, local_rank, config):
    """The chunk manager for a config: symmetric (NVSwitch multicast / peer-mapped)
    fp16 memory when a fused transport is asked for.  Every rank must end up with
    the same kind, so the ranks agree on whether the symmetric set-up worked."""
    world = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
    want = resolve_collectives(parsed["fused_collectives"], world)
    kw = dict(rank=local_rank, default_chunk_size=parsed["default_chunk_size"],
              config=(config or {}).get("client", None))
    return ChunkClient(symmetric=want in _SYMMETRIC_FORMS, **kw), want


def initialize_engine(model_func, local_rank, config=None, client=None):
    """runtime/__init__.py:40-93.  Returns ``(engine, optimizer)``."""
    collectives = None
    if isinstance(model_func, torch.nn.Module):
        assert client is not None, "Must pass the client when passing a nn.Module."
        model = model_func
    else:
        assert callable(model_func), "model_func need to be callable."
        parsed = parse_config(config)
        client, collectives = _client_for(parsed, local_rank, config)
        model = model_func()
        model.to(dtype=torch.float16)
        client.register_module(model)
        # use_hybrid_adam (the reference's default): as many chunk states in HBM as the memory
        # left over allows, the rest in pinned host memory, re-decided every step
        budget = "auto" if parsed["optim_params"].get("use_hybrid_adam", True) else None
        try:
            client.allocate(state_budget_bytes=budget)
            ok = 1
        except RuntimeError:
            if not client.symmetric:
                raise
            ok = 0
        if client.symmetric and client.world_size > 1:
            t = torch.tensor([ok], dtype=torch.int32, device=client.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
            if int(t.item()) == 0:
                # symmetric memory did not come up everywhere: plain memory, NCCL collectives
                client = ChunkClient(rank=local_rank, default_chunk_size=parsed["default_chunk_size"],
                                     config=(config or {}).get("client", None))
                client.register_module(model)
                client.allocate(state_budget_bytes=budget)
                collectives = "nccl"
    engine = ChunkStepEngine(model=model, client=client, config=config, collectives=collectives)
    return (engine, engine.optimizer)
