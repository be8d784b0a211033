"""Model hub: local cache layout, registry of known checkpoints, sha256-verified downloads, HF config parsing.

The machines this framework targets may have no network; ``download_weights`` / ``hf_download_model`` therefore resolve from the
cache first and raise :class:`HubOffline` (with the URL that would have been fetched) when a file is missing and the network is
unreachable or disabled (``FT_HUB_OFFLINE=1``).

Reference parity: ferrotorch-hub/src/{registry.rs:58-1117, download.rs:26, cache.rs:78, hf_config.rs:51, lib.rs:213-424}.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
import shutil
import urllib.parse
import urllib.request
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

from ..errors import FerrotorchError, InvalidArgument


class HubOffline(FerrotorchError):
    pass


def hf_token() -> Optional[str]:
    t = os.environ.get("HF_TOKEN")
    if t:
        return t
    p = Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface")) / "token"
    return p.read_text().strip() if p.exists() else None


class HubCache:
    """``<root>/<repo with / -> -->/<file>`` layout with sha256 sidecars."""

    def __init__(self, root=None):
        self.root = Path(root or os.environ.get("FT_HUB_CACHE", Path.home() / ".cache" / "ferrotorch_b200" / "hub"))
        self.root.mkdir(parents=True, exist_ok=True)

    def path(self, repo: str, filename: str) -> Path:
        return self.root / repo.replace("/", "--") / filename

    def has(self, repo: str, filename: str) -> bool:
        return self.path(repo, filename).exists()

    def put(self, repo: str, filename: str, src) -> Path:
        dst = self.path(repo, filename)
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
        (dst.parent / (dst.name + ".sha256")).write_text(sha256_file(dst))
        return dst

    def verify(self, repo: str, filename: str, expected: Optional[str] = None) -> bool:
        p = self.path(repo, filename)
        if not p.exists():
            return False
        want = expected or ((p.parent / (p.name + ".sha256")).read_text().strip() if (p.parent / (p.name + ".sha256")).exists() else None)
        return want is None or sha256_file(p) == want

    def list(self) -> List[str]:  # noqa: A003
        return sorted(d.name.replace("--", "/") for d in self.root.iterdir() if d.is_dir())

    def clear(self, repo: Optional[str] = None) -> None:
        target = self.root / repo.replace("/", "--") if repo else self.root
        if target.exists():
            shutil.rmtree(target)
        self.root.mkdir(parents=True, exist_ok=True)


def sha256_file(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


class WeightsFormat(enum.Enum):
    """ferrotorch-hub/src/registry.rs:9."""
    SafeTensors = "safetensors"
    FerrotorchStateDict = "ferrotorch_state_dict"


class EntryKind(enum.Enum):
    """A registry row is a usable model or a small fixture kept for tests (registry.rs:26)."""
    Model = "model"
    Fixture = "fixture"


@dataclass
class ModelInfo:
    name: str
    repo: str
    files: List[str]
    family: str
    params: Optional[int] = None
    sha256: Dict[str, str] = field(default_factory=dict)
    description: str = ""
    weights_format: WeightsFormat = WeightsFormat.SafeTensors
    kind: EntryKind = EntryKind.Model


def default_cache_dir() -> Path:
    """``$FT_HUB_CACHE`` or ``~/.cache/ferrotorch_b200/hub`` (the reference keeps ``~/.ferrotorch/hub``; cache.rs:14)."""
    return Path(os.environ.get("FT_HUB_CACHE", Path.home() / ".cache" / "ferrotorch_b200" / "hub"))


def with_auth(req: urllib.request.Request) -> urllib.request.Request:
    """Adds ``Authorization: Bearer <token>`` when a Hugging Face token is configured (auth.rs:64)."""
    tok = hf_token()
    if tok:
        req.add_header("Authorization", f"Bearer {tok}")
    return req


_REGISTRY: Dict[str, ModelInfo] = {m.name: m for m in [
    ModelInfo("llama3-8b", "meta-llama/Meta-Llama-3-8B", ["config.json", "model.safetensors.index.json", "tokenizer.json"], "llama", 8_030_261_248),
    ModelInfo("llama3.3-70b-instruct", "meta-llama/Llama-3.3-70B-Instruct", ["config.json", "model.safetensors.index.json", "tokenizer.json"], "llama", 70_553_706_496),
    ModelInfo("resnet18", "timm/resnet18.tv_in1k", ["model.safetensors"], "resnet", 11_689_512),
    ModelInfo("resnet50", "timm/resnet50.tv_in1k", ["model.safetensors"], "resnet", 25_557_032),
    ModelInfo("vit_b_16", "google/vit-base-patch16-224", ["model.safetensors", "config.json"], "vit", 86_567_656),
    ModelInfo("bert-base-uncased", "google-bert/bert-base-uncased", ["model.safetensors", "config.json", "tokenizer.json"], "bert", 109_482_240),
    ModelInfo("all-MiniLM-L6-v2", "sentence-transformers/all-MiniLM-L6-v2", ["model.safetensors", "config.json", "tokenizer.json"], "bert", 22_713_216),
    ModelInfo("whisper-tiny", "openai/whisper-tiny", ["model.safetensors", "config.json"], "whisper", 37_760_640),
    ModelInfo("stable-diffusion-v1-5", "stable-diffusion-v1-5/stable-diffusion-v1-5", ["unet/diffusion_pytorch_model.safetensors", "vae/diffusion_pytorch_model.safetensors",
              "text_encoder/model.safetensors"], "diffusion", 1_066_235_307),
    ModelInfo("pythia-70m", "EleutherAI/pythia-70m", ["model.safetensors", "config.json", "tokenizer.json"], "gpt_neox", 70_426_624),
]}


def list_models(family: Optional[str] = None) -> List[ModelInfo]:
    return [m for m in _REGISTRY.values() if family is None or m.family == family]


# -- Hugging Face Hub discovery (ferrotorch-hub/src/discovery.rs) --------------------------------------------------------------------------
HUB_BASE = "https://huggingface.co"


@dataclass(frozen=True)
class HfRepoFile:
    rfilename: str


@dataclass
class HfModelSummary:
    """One row of a Hub search (discovery.rs:53). ``author`` falls back to the namespace of ``model_id``."""
    model_id: str
    author: Optional[str] = None
    downloads: Optional[int] = None
    likes: Optional[int] = None
    tags: List[str] = field(default_factory=list)
    library_name: Optional[str] = None
    pipeline_tag: Optional[str] = None

    @classmethod
    def from_json(cls, d: dict):
        mid = d.get("modelId", d.get("id"))
        if not isinstance(mid, str):
            raise InvalidArgument("ferrotorch-hub: failed to parse Hub response: no modelId / id")
        kw = dict(model_id=mid, author=d.get("author") or (mid.split("/", 1)[0] if "/" in mid else None), downloads=d.get("downloads"),
                  likes=d.get("likes"), tags=list(d.get("tags") or []), library_name=d.get("library_name"), pipeline_tag=d.get("pipeline_tag"))
        if cls is HfModelInfo:
            kw["siblings"] = [HfRepoFile(f["rfilename"]) for f in d.get("siblings") or [] if isinstance(f, dict) and "rfilename" in f]
        return cls(**kw)


@dataclass
class HfModelInfo(HfModelSummary):
    """A repository's metadata with its file list (discovery.rs:88)."""
    siblings: List[HfRepoFile] = field(default_factory=list)

    def filenames(self) -> List[str]:
        return [f.rfilename for f in self.siblings]


@dataclass(frozen=True)
class SearchQuery:
    """Builder of a ``/api/models`` query (discovery.rs:123-200)."""
    search: Optional[str] = None
    pipeline_tag: Optional[str] = None
    library: Optional[str] = None
    limit: Optional[int] = None
    sort: Optional[str] = None

    def _with(self, **kw):
        import dataclasses
        return dataclasses.replace(self, **kw)

    def with_search(self, v: str): return self._with(search=v)                        # noqa: E704
    def with_pipeline_tag(self, v: str): return self._with(pipeline_tag=v)            # noqa: E704
    def with_library(self, v: str): return self._with(library=v)                      # noqa: E704
    def with_limit(self, v: int): return self._with(limit=int(v))                     # noqa: E704
    def with_sort(self, v: str): return self._with(sort=v)                            # noqa: E704

    def to_query_string(self) -> str:
        enc = lambda t: urllib.parse.quote(t, safe="-_.~")                            # noqa: E731
        parts = [f"{k}={enc(v)}" for k, v in (("search", self.search), ("pipeline_tag", self.pipeline_tag), ("library", self.library)) if v is not None]
        if self.limit is not None:
            parts.append(f"limit={self.limit}")
        if self.sort is not None:
            parts.append(f"sort={enc(self.sort)}")
        return "/api/models" + ("?" + "&".join(parts) if parts else "")


def _http_get_json(url: str, timeout: float = 30.0):
    if os.environ.get("FT_HUB_OFFLINE") == "1":
        raise HubOffline(f"FT_HUB_OFFLINE=1; would fetch {url}")
    try:
        with urllib.request.urlopen(with_auth(urllib.request.Request(url)), timeout=timeout) as r:
            return json.loads(r.read().decode("utf-8"))
    except OSError as e:
        raise HubOffline(f"cannot reach {url}: {e}") from e
    except ValueError as e:
        raise InvalidArgument(f"ferrotorch-hub: failed to parse Hub response ({url}): {e}") from None


def search_models(query) -> list:
    """A string searches the built-in registry (name, repository, family). A :class:`SearchQuery` asks the Hugging Face Hub and returns
    :class:`HfModelSummary` rows (discovery.rs:222); without network that raises :class:`HubOffline`."""
    if isinstance(query, SearchQuery):
        rows = _http_get_json(HUB_BASE + query.to_query_string())
        if not isinstance(rows, list):
            raise InvalidArgument("ferrotorch-hub: failed to parse Hub search response: expected a list")
        return [HfModelSummary.from_json(r) for r in rows]
    q = query.lower()
    return [m for m in _REGISTRY.values() if q in m.name.lower() or q in m.repo.lower() or q in m.family]


def get_model(repo_id: str) -> HfModelInfo:
    """Hub metadata of one repository, file list included (discovery.rs:261)."""
    if not repo_id:
        raise InvalidArgument("get_model: repo_id must not be empty")
    return HfModelInfo.from_json(_http_get_json(f"{HUB_BASE}/api/models/{repo_id}"))


def get_model_info(name: str) -> Optional[ModelInfo]:
    """Registry row by name, ``None`` when unknown (registry.rs:1122); :func:`model_info` is the raising form."""
    return _REGISTRY.get(name)


def register_model(info: ModelInfo) -> None:
    _REGISTRY[info.name] = info


def model_info(name: str) -> ModelInfo:
    if name not in _REGISTRY:
        raise InvalidArgument(f"unknown model {name!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


def download_weights(repo: str, filename: str, cache: Optional[HubCache] = None, sha256: Optional[str] = None, timeout: float = 30.0) -> Path:
    cache = cache or HubCache()
    if cache.has(repo, filename) and cache.verify(repo, filename, sha256):
        return cache.path(repo, filename)
    url = f"https://huggingface.co/{repo}/resolve/main/{filename}"
    if os.environ.get("FT_HUB_OFFLINE") == "1":
        raise HubOffline(f"{repo}/{filename} is not in the cache ({cache.root}) and FT_HUB_OFFLINE=1; would fetch {url}")
    req = urllib.request.Request(url)
    tok = hf_token()
    if tok:
        req.add_header("Authorization", f"Bearer {tok}")
    dst = cache.path(repo, filename)
    dst.parent.mkdir(parents=True, exist_ok=True)
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r, open(str(dst) + ".part", "wb") as f:
            shutil.copyfileobj(r, f)
    except OSError as e:
        raise HubOffline(f"cannot reach {url}: {e}") from e
    os.replace(str(dst) + ".part", dst)
    got = sha256_file(dst)
    if sha256 and got != sha256:
        dst.unlink()
        raise InvalidArgument(f"sha256 mismatch for {repo}/{filename}: {got} != {sha256}")
    (dst.parent / (dst.name + ".sha256")).write_text(got)
    return dst


def hf_download_model(repo: str, files: Optional[List[str]] = None, cache: Optional[HubCache] = None) -> Path:
    cache = cache or HubCache()
    for f in files or ["config.json", "model.safetensors"]:
        download_weights(repo, f, cache)
    return cache.path(repo, "").parent / repo.replace("/", "--")


@dataclass
class HfTransformerConfig:
    model_type: str = ""
    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: Optional[int] = None
    intermediate_size: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 0
    rms_norm_eps: Optional[float] = None
    layer_norm_eps: Optional[float] = None
    rope_theta: Optional[float] = None
    tie_word_embeddings: bool = False
    raw: dict = field(default_factory=dict)

    @staticmethod
    def from_file(path) -> "HfTransformerConfig":
        return HfTransformerConfig.from_dict(json.loads(Path(path).read_text()))

    @staticmethod
    def from_dict(d: dict) -> "HfTransformerConfig":
        alias = {"n_embd": "hidden_size", "n_layer": "num_hidden_layers", "n_head": "num_attention_heads", "d_model": "hidden_size",
                 "encoder_layers": "num_hidden_layers", "encoder_attention_heads": "num_attention_heads", "n_positions": "max_position_embeddings",
                 "layer_norm_epsilon": "layer_norm_eps", "encoder_ffn_dim": "intermediate_size"}
        keys = set(HfTransformerConfig.__dataclass_fields__) - {"raw"}
        kw = {}
        for k, v in d.items():
            k2 = alias.get(k, k)
            if k2 in keys and k2 not in kw:
                kw[k2] = v
        return HfTransformerConfig(raw=d, **kw)


def load_pretrained(name: str, cache: Optional[HubCache] = None, device="cpu", dtype=None):
    """Resolve a registered model from the cache (downloading if possible) and return ``(config, state_dict)``."""
    from ..serialize import load_safetensors, load_safetensors_sharded
    info = model_info(name)
    cache = cache or HubCache()
    paths = {f: download_weights(info.repo, f, cache, info.sha256.get(f)) for f in info.files}
    cfg = HfTransformerConfig.from_file(paths["config.json"]) if "config.json" in paths else None
    if "model.safetensors.index.json" in paths:
        idx = json.loads(paths["model.safetensors.index.json"].read_text())
        for shard in sorted(set(idx["weight_map"].values())):
            download_weights(info.repo, shard, cache)
        sd = load_safetensors_sharded(paths["model.safetensors.index.json"], dtype, device)
    else:
        st = next(p for f, p in paths.items() if f.endswith(".safetensors"))
        sd = load_safetensors(st, dtype, device)
    return cfg, sd
