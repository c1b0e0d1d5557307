"""bench.py's answers that need no GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm, where the reference is neither built nor to be found, says so in one JSON line and exits with 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, **(env or {})))
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_refused_with_one_line():
    rc, lines = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 2 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and "single-GPU" in d["error"]


def test_reference_arm_without_a_build_says_why(tmp_path):
    """With no built reference and no sources to build it from, the arm prints its one `unavailable` line (the
    real arm runs baseline/_ref/cuda/ref_bench, the unmodified reference built by baseline/build_reference.py)."""
    rc, lines = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1",
                     env={"FORGE_REFERENCE_BUILD": str(tmp_path / "nothing"), "FORGE_REFERENCE_SOURCE": str(tmp_path / "absent")})
    assert rc == 0 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "not built" in d["unavailable"] and "\n" not in d["unavailable"]


def test_the_design_option_keeps_to_one_gpu_and_counts_its_shapes():
    rc, lines = _run("--design", "zatupel", "--gpus", "2")
    assert rc == 2 and len(lines) == 1 and "single-GPU" in json.loads(lines[0])["error"]
    # the shapes it measures are configurations that load, and their matrices are counted from the configuration alone
    sys.path.insert(0, ROOT)
    import bench
    from forge_b200.config import config_from_dict
    z = dict(width=256, layers=4, heads=8, kv_heads=2, dim=32, ff=512, state_heads=4, state_dim=32, rank=16, window=64, vocab=300)
    cfg = config_from_dict(bench.zatupel_shape(**z))
    assert [l["type"] for l in cfg.layers] == ["attention", "wkv", "attention", "general_delta"]
    layers, head = bench.zatupel_matmul_params(cfg)
    att = 256 * (8 * 32 + 2 * 32 + 2 * 32 + 8) + 256 * 8 * 32
    state = lambda n: 256 * 128 * n + 16 * (256 + 128)
    assert layers == 2 * att + state(5) + state(6) + 4 * 3 * 256 * 512 and head == 300 * 256


def test_the_other_design_option_too():
    rc, lines = _run("--design", "tidenex", "--gpus", "2")
    assert rc == 2 and len(lines) == 1 and "single-GPU" in json.loads(lines[0])["error"]
    sys.path.insert(0, ROOT)
    import bench
    import torch
    from forge_b200.config import config_from_dict
    from forge_b200.engine.model import Model
    from forge_b200.parts import Runtime
    z = dict(width=256, layers=3, heads=8, kv_heads=2, dim=32, ff=512, state_heads=4, state_dim=32, rank=16, window=64, vocab=300)
    cfg = config_from_dict(bench.tidenex_shape(**z))
    assert [l["type"] for l in cfg.layers] == ["attention", "attention", "parallel"] and cfg.loop is None
    layers, head = bench.tidenex_matmul_params(cfg)
    # counted from the configuration alone, the matrices are what the model's own tensor list holds (the head is the embedding)
    specs = Model(cfg.plan(), Runtime(torch.device("cpu"), torch.bfloat16)).tensor_specs()
    matrices = sum(s.shape[0] * s.shape[1] for n, s in specs.items() if len(s.shape) == 2 and s.required and n != "embed")
    assert layers == matrices and head == 300 * 256


def test_the_third_design_option_too():
    rc, lines = _run("--design", "tuzavik", "--gpus", "2")
    assert rc == 2 and len(lines) == 1 and "single-GPU" in json.loads(lines[0])["error"]
    sys.path.insert(0, ROOT)
    import bench
    import torch
    from forge_b200.config import config_from_dict
    from forge_b200.engine.model import Model
    from forge_b200.parts import Runtime
    z = dict(width=256, layers=5, heads=8, kv_heads=2, dim=32, ff=512, state_heads=4, state_dim=32, rank=16, window=64, vocab=300)
    cfg = config_from_dict(bench.tuzavik_shape(**z))
    assert [l["type"] for l in cfg.layers] == ["latent_attention", "retention", "retention", "latent_attention", "latent_attention"]
    assert [l["mixer"].get("kv_from") for l in cfg.layers] == [None, None, None, 0, None]
    assert [l["mlp"]["kind"] for l in cfg.layers] == ["dense", "moe", "dense", "moe", "dense"]
    # counted from the configuration alone with every expert read, the matrices are what the model's own tensor list holds
    layers, head = bench.tuzavik_matmul_params(cfg, experts_read=8)
    specs = Model(cfg.plan(), Runtime(torch.device("cpu"), torch.bfloat16)).tensor_specs()
    matrices = sum(s.shape[0] * s.shape[1] for n, s in specs.items() if len(s.shape) == 2 and s.required and n not in ("embed", "bigram", "head"))
    assert layers == matrices and head == 300 * 256
    per_token, _ = bench.tuzavik_matmul_params(cfg)
    assert layers - per_token == 2 * 6 * 3 * 256 * 256                    # six of eight experts of two routed layers


def test_the_fourth_design_option_too():
    rc, lines = _run("--design", "natalorn", "--gpus", "2")
    assert rc == 2 and len(lines) == 1 and "single-GPU" in json.loads(lines[0])["error"]
    sys.path.insert(0, ROOT)
    import bench
    import torch
    from forge_b200.config import config_from_dict
    from forge_b200.engine.model import Model
    from forge_b200.parts import Runtime
    z = dict(width=256, layers=5, heads=8, kv_heads=2, dim=32, ff=512, state_heads=4, state_dim=32, rank=16, window=64, vocab=300)
    cfg = config_from_dict(bench.natalorn_shape(**z))
    assert [l["type"] for l in cfg.layers] == ["attention", "latent_attention", "attention", "attention_2", "attention"] and cfg.streams == 4
    # counted from the configuration alone with every expert read, the matrices are what the model's own tensor list holds
    layers, head = bench.natalorn_matmul_params(cfg, experts_read=8)
    specs = Model(cfg.plan(), Runtime(torch.device("cpu"), torch.bfloat16)).tensor_specs()
    matrices = sum(s.shape[0] * s.shape[1] for n, s in specs.items() if len(s.shape) == 2 and s.required and n not in ("embed", "head") and ".hc" not in n)
    assert layers == matrices and head == 300 * 256
    per_token, _ = bench.natalorn_matmul_params(cfg)
    assert layers - per_token == 5 * 6 * 3 * 256 * 128                    # six of eight experts of five routed layers
    assert bench._visible_pairs(10, window=4) == 1 + 2 + 3 + 7 * 4 and bench._visible_pairs(10, chunk=4) == 10 + 10 + 3
