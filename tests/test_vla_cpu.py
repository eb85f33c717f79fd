"""GR00T-N1.5-shaped model end to end (prefill feeding the action head in ONE profile): structure checks on CPU."""
import dataclasses
import json

from aginfer_b200 import planfmt
from aginfer_b200.recipes import dit, lowering, vla
from aginfer_b200.target import CudaArch
from tests.test_qwen_vl_cpu import table


def inventory(cfg):
    return {**table(cfg.backbone), **{k: ("BF16", v) for k, v in dit.weight_shapes(cfg.head).items()}}


def test_one_profile_from_pixels_to_actions():
    cfg = vla.VlaConfig()                       # BASELINE config 4 backbone + config 3 head, full depth
    r = vla.build_recipe(cfg, inventory(cfg), packed=True)
    plan = r.plan()
    compiled = planfmt.compile_execution_plan(plan, CudaArch.SM100, weight_size=r.weight_bytes)
    assert compiled.input_names == ("pixels", "input_ids", "positions", "state", "noise")
    assert compiled.output_names == ("hidden_out", "kv_cache", "status", "actions")
    assert len(plan["shape_dispatch"]) == 1 and plan["cuda_graph_templates"] == [{"profile": "default"}]
    launches = plan["shape_dispatch"][0]["launches"]
    # the head's context is the prefill's output tensor: some launch after the final norm reads it as an argument
    hidden = [i for i, l in enumerate(launches) if any(a.get("tensor") == "hidden_out" for a in l["arguments"])]
    assert len(hidden) >= 2 and launches[hidden[0]]["kernel"].startswith("agi_rmsnorm")
    assert sum(l["kernel"] == "agi_euler_step" for l in launches) == cfg.head.steps
    used = {a["weights_offset"] for l in launches for a in l["arguments"] if "weights_offset" in a}
    assert used >= {off for name, off in r.weight_offsets.items() if name.startswith("action_head.")}


def test_a_head_that_does_not_fit_the_backbone_is_refused():
    try:
        vla.VlaConfig(head=dit.DitConfig(backbone_tokens=300))
        raise AssertionError("expected a ValueError")
    except ValueError as exc:
        assert "288 tokens" in str(exc)


def test_lowering_picks_the_joint_recipe_for_a_joint_checkpoint():
    cfg = vla.reduced()
    graph = {"passes": ["fuse_qkv", "fuse_mlp", "fuse_norm"], "subgraphs": ["vision", "vlm_conditioning", "flow_matching_dit_step"]}
    config = {"aginfer_recipe": {"config": json.loads(json.dumps(dataclasses.asdict(cfg)))}}
    recipe, name, shape = lowering.lower("groot_n1_5", graph, inventory(cfg), config, {"profiles": [{}]})
    assert name == "vla" and shape["head"]["backbone_tokens"] == 288 and shape["backbone"]["layers"] == 2
    assert recipe.plan() == vla.build_recipe(cfg, inventory(cfg)).plan()
