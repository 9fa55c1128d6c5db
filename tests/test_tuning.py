"""The configuration search and its cache (CPU, stand-in engines), and on the GPU both embedders tuned for real."""
import json

import pytest
import torch

from ittai_b200 import tuning

gpu = pytest.mark.gpu


def test_fastest_valid_candidate_is_cached(tmp_path):
    path = str(tmp_path / "tune.json")
    cands = [{"v": "slow"}, {"v": "wrong"}, {"v": "fast"}, {"v": "broken"}]
    built, log = [], []

    def build(c):
        if c["v"] == "broken":
            raise ValueError("cannot build")
        built.append(c["v"])
        return c

    cos = {"slow": 0.9999, "wrong": 0.95, "fast": 0.9995}
    ms = {"slow": 3.0, "fast": 1.0}
    best = tuning.choose("gpu|model|64", cands, build, lambda e: cos[e["v"]], lambda e: ms[e["v"]], path=path, log=log.append)
    assert best == {"v": "fast"} and built == ["slow", "wrong", "fast"]
    assert any("MISMATCH" in m for m in log) and any("failed (ValueError" in m for m in log)
    assert json.load(open(path)) == {"gpu|model|64": {"v": "fast"}}
    # the second call does not build anything
    again = tuning.choose("gpu|model|64", cands, lambda c: 1 / 0, None, None, path=path)
    assert again == {"v": "fast"}
    # another key is searched and added beside the first
    tuning.choose("gpu|model|8", cands[:1], build, lambda e: 1.0, lambda e: 2.0, path=path, log=log.append)
    assert set(json.load(open(path))) == {"gpu|model|64", "gpu|model|8"}


def test_no_valid_candidate_fails(tmp_path):
    with pytest.raises(RuntimeError, match="no kernel configuration"):
        tuning.choose("k", [{"a": 1}], lambda c: c, lambda e: 0.5, lambda e: 1.0, path=str(tmp_path / "t.json"), log=lambda m: None)


@gpu
def test_embedders_tune_against_the_eager_modules(tiny_hf, tmp_path):
    from ittai_b200.qwen3 import Qwen3Embedder
    from ittai_b200.siglip.kernel import Siglip2Embedder
    from oracle import siglip_hf
    model, dims = tiny_hf
    model = model.to("cuda")
    try:
        emb = Qwen3Embedder(model, max_tokens=8192, max_seqs=64, tune=False)
        choice = emb._tune(path=str(tmp_path / "q.json"))
        assert choice in list(Qwen3Embedder.CANDIDATES)
    finally:
        model.to("cpu")
    vm = siglip_hf.build_hf(seed=2, device="cuda", n_layers=2)
    se = Siglip2Embedder(vm, batch_size=4, tune=False)
    choice = se._tune("vit-b16-test", path=str(tmp_path / "s.json"))
    assert choice in list(Siglip2Embedder.CANDIDATES)
    assert list(json.load(open(tmp_path / "s.json"))) == [f"{torch.cuda.get_device_name()}|vit-b16-test|4"]
