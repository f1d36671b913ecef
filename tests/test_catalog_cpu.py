"""Catalog lookup, the cache store and name resolution (no network)."""
import json

import pytest

from hartsyinference_b200.assets.catalog import (CatalogEntry, ModelCacheStore, ModelCatalog, ModelResolver,
                                                 hf_hub_snapshot)
from hartsyinference_b200.engine.requests import Modality
from hartsyinference_b200.exceptions import UnsupportedModelError


def test_catalog_lookup(tmp_path):
    cat = ModelCatalog()
    assert cat.find("flux-dev").id == "flux.1-dev" and cat.find("Black-Forest-Labs/FLUX.1-dev").id == "flux.1-dev"
    assert cat.find("LLAMA-3-70B").repo == "meta-llama/Llama-3.3-70B-Instruct" and cat.find("nope") is None
    assert {e.modality for e in cat.entries()} >= {Modality.TEXT, Modality.IMAGE, Modality.VIDEO, Modality.TRANSCRIBE}
    assert all(e.modality == Modality.VIDEO for e in cat.entries(Modality.VIDEO)) and cat.entries(Modality.VIDEO)
    extra = tmp_path / "extra.json"
    extra.write_text(json.dumps([{"id": "my-model", "modality": "text", "family": "llama", "repo": "me/my-model", "aliases": ["mm"]}]))
    cat2 = ModelCatalog(extra_file=extra)
    assert cat2.find("mm").repo == "me/my-model"


def test_store_and_resolver(tmp_path):
    ckpt = tmp_path / "src" / "tiny"
    ckpt.mkdir(parents=True)
    (ckpt / "config.json").write_text(json.dumps({"model_type": "qwen2"}))
    (ckpt / "model.safetensors").write_bytes(b"\0" * 100)
    store = ModelCacheStore(tmp_path / "store")
    assert store.list() == [] and store.path_of("qwen2.5-0.5b-instruct") is None
    dst = store.add_local("qwen2.5-0.5b-instruct", ckpt)
    assert dst.is_symlink() and (dst / "config.json").exists()
    with pytest.raises(FileExistsError):
        store.add_local("qwen2.5-0.5b-instruct", ckpt)
    listed = store.list()
    assert listed[0]["id"] == "qwen2.5-0.5b-instruct" and listed[0]["bytes"] > 100 and listed[0]["source"] == "local"

    # a repository that only exists in a Hugging Face hub cache
    snap = tmp_path / "hub" / "models--openai--whisper-tiny" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text(json.dumps({"model_type": "whisper"}))
    assert hf_hub_snapshot("openai/whisper-tiny", tmp_path / "hub") == snap

    res = ModelResolver(store=store, hub_dir=tmp_path / "hub")
    s = res.resolve("qwen2.5-0.5b")                       # alias -> catalog -> store
    assert s.catalog == "qwen2.5-0.5b-instruct" and s.local_path == str(dst) and s.modality == Modality.TEXT
    s = res.resolve("whisper-tiny")                       # catalog -> hub cache
    assert s.local_path == str(snap) and s.modality == Modality.TRANSCRIBE
    s = res.resolve("openai/whisper-tiny")                # bare repository id
    assert s.local_path == str(snap)
    s = res.resolve(str(ckpt))                            # a path resolves to itself
    assert s.local_path == str(ckpt) and s.catalog is None
    assert res.resolve("synthetic:flux-tiny", Modality.IMAGE).local_path is None
    with pytest.raises(UnsupportedModelError) as e:
        res.resolve("flux-dev")
    assert "pull flux.1-dev" in str(e.value) and "gated" in str(e.value)

    # side models that are on disk are attached by role
    t5 = tmp_path / "src" / "t5"
    t5.mkdir()
    store.add_local("t5-xxl", t5)
    flux = tmp_path / "src" / "flux"
    flux.mkdir()
    store.add_local("flux.1-schnell", flux, link=False)
    s = res.resolve("flux-schnell")
    assert s.modality == Modality.IMAGE and s.aux == {"text_encoder": str(store.path_of("t5-xxl"))}
    assert store.remove("flux.1-schnell") and store.path_of("flux.1-schnell") is None and not store.remove("flux.1-schnell")
    assert ckpt.exists()                                   # removing a link never touches its target
    assert store.remove("qwen2.5-0.5b-instruct") and ckpt.exists()


def test_cli_pull_from_disk_and_list(tmp_path):
    from click.testing import CliRunner
    from hartsyinference_b200.cli.main import cli
    src = tmp_path / "w"
    src.mkdir()
    (src / "config.json").write_text("{}")
    r = CliRunner().invoke(cli, ["pull", "whisper-tiny", "--from", str(src), "--dir", str(tmp_path / "store")])
    assert r.exit_code == 0, r.output
    r = CliRunner().invoke(cli, ["models", "--dir", str(tmp_path / "store")])
    assert r.exit_code == 0 and "whisper-tiny" in r.output
    r = CliRunner().invoke(cli, ["models", "--catalog"])
    assert r.exit_code == 0 and "flux.1-dev" in r.output and "black-forest-labs/FLUX.1-dev" in r.output


def test_recipe_defaults_fill_untouched_fields():
    from hartsyinference_b200.engine.diffusion_service import apply_recipe_defaults
    from hartsyinference_b200.engine.requests import ImageRequest, ModelSpec
    spec = ModelSpec("flux-schnell", Modality.IMAGE, catalog="flux.1-schnell")
    r = apply_recipe_defaults(spec, ImageRequest(prompt="x"))
    assert (r.steps, r.guidance) == (4, 0.0) and r.prompt == "x"
    r = apply_recipe_defaults(spec, ImageRequest(prompt="x", steps=9))
    assert r.steps == 9 and r.guidance == 0.0                 # what the caller set stays
    same = ImageRequest(prompt="y")
    assert apply_recipe_defaults(ModelSpec("/some/path", Modality.IMAGE), same) is same
