"""Model catalog, local cache store and name resolution.

``ModelCatalog`` lists the checkpoints the engine knows by id (repository, files, modality, family
and the family's default request parameters). ``ModelCacheStore`` is the on-disk store
(``<root>/<id>/...`` plus a small JSON index) that ``pull`` fills and ``list`` reads.
``ModelResolver`` turns whatever a caller wrote (a path, a catalog id or alias, a Hugging Face
repository id) into a ``ModelSpec`` with a local path, looking in the store and in the Hugging Face
hub cache; it never reaches for the network by itself.

Reference: src/HartsyInference.Engine/Registry/ (ModelCatalog, ModelRegistry, ModelResolver,
ModelCacheStore) and src/HartsyInference.Engine/HuggingFace/.
"""
from __future__ import annotations

import json
import os
import shutil
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

from ..engine.requests import Modality, ModelSpec
from ..exceptions import UnsupportedModelError


@dataclass(frozen=True)
class CatalogEntry:
    id: str
    modality: Modality
    family: str                                   # llama, qwen2, deepseek3, flux, wan, whisper, clip, bert, llava ...
    repo: str                                     # Hugging Face repository id
    files: tuple = ()                             # patterns to fetch; empty = whole repository
    aliases: tuple = ()
    aux: dict = field(default_factory=dict)       # side models by role -> catalog id (vae, text_encoder, ...)
    defaults: dict = field(default_factory=dict)  # request defaults of the family (steps, guidance, ...)
    params_b: float = 0.0                         # parameters in billions (placement planning)
    license: str = ""
    gated: bool = False


def _e(*a, **k) -> CatalogEntry:
    return CatalogEntry(*a, **k)


BUILTIN: tuple = (
    _e("qwen2.5-0.5b-instruct", Modality.TEXT, "qwen2", "Qwen/Qwen2.5-0.5B-Instruct", aliases=("qwen2.5-0.5b",), params_b=0.49, license="apache-2.0"),
    _e("qwen2.5-7b-instruct", Modality.TEXT, "qwen2", "Qwen/Qwen2.5-7B-Instruct", params_b=7.6, license="apache-2.0"),
    _e("qwen3-8b", Modality.TEXT, "qwen3", "Qwen/Qwen3-8B", params_b=8.2, license="apache-2.0"),
    _e("qwen3-30b-a3b", Modality.TEXT, "qwen3_moe", "Qwen/Qwen3-30B-A3B", params_b=30.5, license="apache-2.0"),
    _e("llama-3.1-8b-instruct", Modality.TEXT, "llama", "meta-llama/Llama-3.1-8B-Instruct", aliases=("llama-3-8b",), params_b=8.0, license="llama3.1", gated=True),
    _e("llama-3.3-70b-instruct", Modality.TEXT, "llama", "meta-llama/Llama-3.3-70B-Instruct", aliases=("llama-3-70b",), params_b=70.6, license="llama3.3", gated=True),
    _e("mistral-7b-instruct", Modality.TEXT, "mistral", "mistralai/Mistral-7B-Instruct-v0.3", params_b=7.2, license="apache-2.0"),
    _e("mixtral-8x7b-instruct", Modality.TEXT, "mixtral", "mistralai/Mixtral-8x7B-Instruct-v0.1", params_b=46.7, license="apache-2.0"),
    _e("gemma-2-2b-it", Modality.TEXT, "gemma2", "google/gemma-2-2b-it", params_b=2.6, license="gemma", gated=True),
    _e("gemma-3-4b-it", Modality.TEXT, "gemma3", "google/gemma-3-4b-it", params_b=4.3, license="gemma", gated=True),
    _e("phi-3.5-mini-instruct", Modality.TEXT, "phi3", "microsoft/Phi-3.5-mini-instruct", params_b=3.8, license="mit"),
    _e("granite-3.0-2b-instruct", Modality.TEXT, "granite", "ibm-granite/granite-3.0-2b-instruct", params_b=2.5, license="apache-2.0"),
    _e("olmo-2-7b-instruct", Modality.TEXT, "olmo2", "allenai/OLMo-2-1124-7B-Instruct", params_b=7.3, license="apache-2.0"),
    _e("deepseek-v3", Modality.TEXT, "deepseek3", "deepseek-ai/DeepSeek-V3", params_b=671.0, license="deepseek"),
    _e("deepseek-r1-distill-qwen-1.5b", Modality.TEXT, "qwen2", "deepseek-ai/DeepSeek-R1-Distill-Qwen-1.5B", params_b=1.8, license="mit"),
    _e("mamba-130m", Modality.TEXT, "mamba", "state-spaces/mamba-130m-hf", params_b=0.13, license="apache-2.0"),
    _e("llava-1.5-7b", Modality.TEXT, "llava", "llava-hf/llava-1.5-7b-hf", params_b=7.1, license="llama2"),
    _e("bge-small-en", Modality.EMBEDDINGS, "bert", "BAAI/bge-small-en-v1.5", params_b=0.033, license="mit"),
    _e("all-minilm-l6", Modality.EMBEDDINGS, "bert", "sentence-transformers/all-MiniLM-L6-v2", params_b=0.023, license="apache-2.0"),
    _e("flux.1-dev", Modality.IMAGE, "flux", "black-forest-labs/FLUX.1-dev", aliases=("flux-dev",), params_b=12.0,
       aux={"text_encoder": "t5-xxl", "clip": "clip-vit-l"}, defaults={"steps": 28, "guidance": 3.5, "width": 1024, "height": 1024},
       license="flux-1-dev-non-commercial", gated=True),
    _e("flux.1-schnell", Modality.IMAGE, "flux", "black-forest-labs/FLUX.1-schnell", aliases=("flux-schnell",), params_b=12.0,
       aux={"text_encoder": "t5-xxl", "clip": "clip-vit-l"}, defaults={"steps": 4, "guidance": 0.0, "width": 1024, "height": 1024},
       license="apache-2.0"),
    _e("wan2.1-t2v-14b", Modality.VIDEO, "wan", "Wan-AI/Wan2.1-T2V-14B-Diffusers", aliases=("wan-14b",), params_b=14.0,
       aux={"text_encoder": "umt5-xxl"}, defaults={"steps": 50, "guidance": 5.0, "width": 832, "height": 480, "frames": 81},
       license="apache-2.0"),
    _e("wan2.1-t2v-1.3b", Modality.VIDEO, "wan", "Wan-AI/Wan2.1-T2V-1.3B-Diffusers", params_b=1.3,
       aux={"text_encoder": "umt5-xxl"}, defaults={"steps": 50, "guidance": 6.0, "width": 832, "height": 480, "frames": 81},
       license="apache-2.0"),
    _e("t5-xxl", Modality.EMBEDDINGS, "t5", "google/t5-v1_1-xxl", params_b=4.7, license="apache-2.0"),
    _e("umt5-xxl", Modality.EMBEDDINGS, "t5", "google/umt5-xxl", params_b=5.7, license="apache-2.0"),
    _e("clip-vit-l", Modality.VISION, "clip", "openai/clip-vit-large-patch14", params_b=0.43, license="mit"),
    _e("clip-vit-l-336", Modality.VISION, "clip", "openai/clip-vit-large-patch14-336", params_b=0.43, license="mit"),
    _e("whisper-tiny", Modality.TRANSCRIBE, "whisper", "openai/whisper-tiny", params_b=0.039, license="apache-2.0"),
    _e("whisper-small", Modality.TRANSCRIBE, "whisper", "openai/whisper-small", params_b=0.24, license="apache-2.0"),
    _e("whisper-large-v3", Modality.TRANSCRIBE, "whisper", "openai/whisper-large-v3", params_b=1.55, license="apache-2.0"),
    _e("whisper-large-v3-turbo", Modality.TRANSCRIBE, "whisper", "openai/whisper-large-v3-turbo", params_b=0.81, license="mit"),
)


class ModelCatalog:
    def __init__(self, entries=BUILTIN, extra_file: Optional[str | Path] = None):
        self._by_id: dict[str, CatalogEntry] = {}
        self._alias: dict[str, str] = {}
        for e in entries:
            self.add(e)
        if extra_file and Path(extra_file).exists():       # user catalog: a JSON list of entries
            for d in json.loads(Path(extra_file).read_text()):
                d["modality"] = Modality(d["modality"])
                for k in ("files", "aliases"):
                    d[k] = tuple(d.get(k, ()))
                self.add(CatalogEntry(**d))

    def add(self, e: CatalogEntry) -> None:
        self._by_id[e.id.lower()] = e
        for a in (e.repo,) + tuple(e.aliases):
            self._alias[a.lower()] = e.id.lower()

    def find(self, name: str) -> Optional[CatalogEntry]:
        n = name.lower()
        return self._by_id.get(n) or self._by_id.get(self._alias.get(n, ""))

    def entries(self, modality: Optional[Modality] = None) -> list[CatalogEntry]:
        return [e for e in self._by_id.values() if modality is None or e.modality == modality]


class ModelCacheStore:
    """``<root>/<id>/`` holds one checkpoint; ``<root>/index.json`` records where it came from."""

    def __init__(self, root: str | Path = "~/.hartsyinference/models"):
        self.root = Path(os.path.expanduser(str(root)))

    def _index_path(self) -> Path:
        return self.root / "index.json"

    def index(self) -> dict:
        p = self._index_path()
        return json.loads(p.read_text()) if p.exists() else {}

    def _write_index(self, idx: dict) -> None:
        self.root.mkdir(parents=True, exist_ok=True)
        tmp = self._index_path().with_suffix(".tmp")
        tmp.write_text(json.dumps(idx, indent=1, sort_keys=True))
        tmp.replace(self._index_path())

    def path_of(self, model_id: str) -> Optional[Path]:
        p = self.root / model_id.lower().replace("/", "--")
        return p if p.exists() else None

    def add_local(self, model_id: str, src: str | Path, link: bool = True, source: str = "local") -> Path:
        """Register a checkpoint that is already on disk (symlink by default, else copy)."""
        src = Path(src).resolve()
        if not src.exists():
            raise FileNotFoundError(src)
        dst = self.root / model_id.lower().replace("/", "--")
        self.root.mkdir(parents=True, exist_ok=True)
        if dst.exists() or dst.is_symlink():
            raise FileExistsError(f"{model_id} is already in the store")
        if link:
            dst.symlink_to(src, target_is_directory=src.is_dir())
        elif src.is_dir():
            shutil.copytree(src, dst)
        else:
            dst.mkdir()
            shutil.copy2(src, dst / src.name)
        idx = self.index()
        idx[model_id.lower()] = {"source": source, "origin": str(src), "added": int(time.time())}
        self._write_index(idx)
        return dst

    def remove(self, model_id: str) -> bool:
        dst = self.root / model_id.lower().replace("/", "--")
        found = dst.exists() or dst.is_symlink()
        if dst.is_symlink() or dst.is_file():
            dst.unlink()
        elif dst.is_dir():
            shutil.rmtree(dst)
        idx = self.index()
        if idx.pop(model_id.lower(), None) is not None:
            self._write_index(idx)
        return found

    def list(self) -> list[dict]:
        out = []
        idx = self.index()
        if not self.root.exists():
            return out
        for p in sorted(self.root.iterdir()):
            if p.name == "index.json" or p.name.endswith(".tmp"):
                continue
            size = sum(f.stat().st_size for f in p.rglob("*") if f.is_file()) if p.is_dir() else p.stat().st_size
            out.append({"id": p.name, "path": str(p), "bytes": size, **idx.get(p.name, {})})
        return out


def hf_hub_snapshot(repo: str, hub_dir: Optional[str | Path] = None) -> Optional[Path]:
    """The newest snapshot of ``repo`` in a Hugging Face hub cache directory, if it was downloaded."""
    hub = Path(hub_dir or os.environ.get("HF_HUB_CACHE") or Path(os.environ.get("HF_HOME", "~/.cache/huggingface")).expanduser() / "hub").expanduser()
    snaps = hub / ("models--" + repo.replace("/", "--")) / "snapshots"
    if not snaps.exists():
        return None
    cands = [p for p in snaps.iterdir() if p.is_dir()]
    return max(cands, key=lambda p: p.stat().st_mtime) if cands else None


class ModelResolver:
    def __init__(self, catalog: Optional[ModelCatalog] = None, store: Optional[ModelCacheStore] = None,
                 hub_dir: Optional[str | Path] = None):
        self.catalog = catalog or ModelCatalog()
        self.store = store or ModelCacheStore()
        self.hub_dir = hub_dir

    def _local(self, entry_or_id) -> Optional[Path]:
        mid = entry_or_id.id if isinstance(entry_or_id, CatalogEntry) else entry_or_id
        p = self.store.path_of(mid)
        if p is not None:
            return p
        repo = entry_or_id.repo if isinstance(entry_or_id, CatalogEntry) else (mid if "/" in mid else None)
        if repo:
            return self.store.path_of(repo) or hf_hub_snapshot(repo, self.hub_dir)
        return None

    def resolve(self, name: str, modality: Optional[Modality] = None) -> ModelSpec:
        """Path -> itself; ``synthetic:*`` -> itself; catalog id / alias / repository id -> the local copy.
        Raises ``UnsupportedModelError`` naming the ``pull`` command when nothing is on disk."""
        if name.startswith("synthetic:"):
            return ModelSpec(name, modality or Modality.TEXT, local_path=None)
        p = Path(os.path.expanduser(name))
        if p.exists():
            return ModelSpec(name, modality or self._guess_modality(p), local_path=str(p))
        entry = self.catalog.find(name)
        local = self._local(entry or name)
        if local is None:
            what = f"'{name}' ({entry.repo})" if entry else f"'{name}'"
            gate = " (gated: needs an access token)" if entry and entry.gated else ""
            raise UnsupportedModelError(f"{what} is not on this machine{gate}; fetch it with `pull {entry.id if entry else name}` "
                                        f"or pass a path")
        spec = ModelSpec(name, modality or (entry.modality if entry else self._guess_modality(local)),
                         catalog=entry.id if entry else None, local_path=str(local))
        if entry:
            for role, aux_id in entry.aux.items():
                aux_entry = self.catalog.find(aux_id)
                aux_local = self._local(aux_entry or aux_id)
                if aux_local is not None:
                    spec.aux[role] = str(aux_local)
        return spec

    @staticmethod
    def _guess_modality(path: Path) -> Modality:
        from .registry import detect
        fam = detect(path).family
        return {"dit-image": Modality.IMAGE, "dit-video": Modality.VIDEO}.get(fam, Modality.TEXT)

    def pull(self, name: str, token: Optional[str] = None) -> Path:
        """Download a catalog entry or repository into the store (needs network access and
        ``huggingface_hub``); returns the local directory."""
        entry = self.catalog.find(name)
        repo = entry.repo if entry else name
        if "/" not in repo:
            raise UnsupportedModelError(f"'{name}' is neither a catalog id nor a repository id")
        try:
            from huggingface_hub import snapshot_download
        except ImportError as e:      # pragma: no cover
            raise UnsupportedModelError("pull needs the huggingface_hub package") from e
        dst = self.store.root / (entry.id if entry else repo.replace("/", "--")).lower()
        snapshot_download(repo, local_dir=str(dst), allow_patterns=list(entry.files) or None if entry else None, token=token)
        idx = self.store.index()
        idx[dst.name] = {"source": "huggingface", "origin": repo, "added": int(time.time())}
        self.store._write_index(idx)
        return dst
