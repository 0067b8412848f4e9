"""initialize_engine's config surface (patrickstar/runtime/engine.py:53-105):
keys, defaults and quirks, as a pure function (no GPU)."""
import pytest

from patrickstar_b200.engine import parse_config


def test_defaults():
    p = parse_config(None)
    assert p["optim_type"] == "Adam"
    assert p["optim_params"] == {"lr": 0.01, "betas": (0.9, 0.999), "eps": 1e-8, "weight_decay": 0,
                                 "use_hybrid_adam": True}
    assert p["scaler"] == "none" and p["gradient_clipping"] == -1
    assert p["default_chunk_size"] == 32 * 1024 * 1024
    assert parse_config({})["optim_params"]["lr"] == 0.01


def test_readme_style_config():
    cfg = {
        "optimizer": {"type": "Adam", "params": {"lr": 0.001, "betas": (0.9, 0.999), "eps": 1e-6,
                                                 "weight_decay": 0, "use_hybrid_adam": True}},
        "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 3, "loss_scale_window": 1000,
                 "hysteresis": 2, "min_loss_scale": 1},
        "default_chunk_size": 64 * 1024 * 1024,
    }
    p = parse_config(cfg)
    assert p["default_chunk_size"] == 64 * 1024 * 1024
    assert p["optim_params"]["eps"] == 1e-6
    kind, kw = p["scaler"]
    # the quirk: "hysteresis" becomes scale_factor; there is no delayed shift
    assert kind == "dynamic" and kw == {"init_scale": 8, "scale_factor": 2, "scale_window": 1000, "min_scale": 1}


def test_missing_params_are_filled_and_adamw_selected():
    p = parse_config({"optimizer": {"type": "AdamW", "params": {"lr": 3e-4}}})
    assert p["optim_type"] == "AdamW" and p["optim_params"]["lr"] == 3e-4
    assert p["optim_params"]["betas"] == (0.9, 0.999) and p["optim_params"]["use_hybrid_adam"] is True


def test_errors_like_the_reference():
    with pytest.raises(ValueError, match="Only support Adam and AdamW"):
        parse_config({"optimizer": {"type": "SGD"}})
    with pytest.raises(AssertionError, match="Must enable fp16"):
        parse_config({"fp16": {"enabled": False, "loss_scale": 0}})
    with pytest.raises(AssertionError, match="loss_scale"):
        parse_config({"fp16": {"enabled": True}})
    assert parse_config({"fp16": {"enabled": True, "loss_scale": 512}})["scaler"] == ("static", 512)
    assert parse_config({"fp16": {"enabled": True, "loss_scale": 0}})["scaler"][1]["init_scale"] == 2 ** 16
    assert parse_config({"gradient_clipping": 1.0})["gradient_clipping"] == 1.0


def test_collectives_key_under_client_opts():
    """client.opts.fused_collectives chooses how a data-parallel step exchanges
    chunks; "auto" resolves by world size."""
    from patrickstar_b200.engine import resolve_collectives
    assert parse_config(None)["fused_collectives"] == "auto"
    assert parse_config({})["fused_collectives"] == "auto"
    cfg = {"client": {"mem_tracer": {"margin_use_ratio": 0.7}, "opts": {"with_mem_saving_comm": False,
                                                                      "fused_collectives": "nccl"}}}
    assert parse_config(cfg)["fused_collectives"] == "nccl"
    with pytest.raises(ValueError, match="fused_collectives"):
        parse_config({"client": {"opts": {"fused_collectives": "ring"}}})
    assert [resolve_collectives("auto", w) for w in (1, 2, 3, 4, 8)] == ["none", "p2p", "p2p", "multimem", "multimem"]
    assert resolve_collectives("nccl", 8) == "nccl" and resolve_collectives("multimem", 2) == "multimem"
