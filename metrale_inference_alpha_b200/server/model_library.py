"""Model library: resolve a model argument to a directory, and download a repository into the
Hugging Face cache layout.

``resolve_model_dir`` accepts a preset name (returned as is), a local checkpoint directory, or a
repository id looked up in the cache (``<cache>/models--org--name/refs/main`` ->
``snapshots/<revision>``), with errors that say what is missing and how to fetch it.

``download`` talks to a Hub-compatible endpoint (``/api/models/<repo>/revision/<rev>`` for the
file list, ``/<repo>/resolve/<rev>/<file>`` for content): it selects metadata and safetensors
files only, refuses names that would escape the snapshot directory, checks free disk space,
fetches small files first, resumes ``.part`` files with a Range request, and publishes
``refs/main`` only after every file is complete, so an interrupted download is never mistaken for
a model. The machine this engine is developed on has no network: the tests serve a repository
from a local HTTP server.

Role of the reference's ``crates/server/src/model_resolver.rs`` and ``model_download/``.
"""
from __future__ import annotations

import json
import os
import shutil
import urllib.error
import urllib.request
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, List, Optional, Tuple

METADATA = ("config.json", "params.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json",
            "tokenizer.model", "special_tokens_map.json", "vocab.json", "merges.txt", "chat_template.jinja",
            "preprocessor_config.json", "processor_config.json", "hf_quant_config.json")
_SKIP_DIRS = ("original/", "onnx/", "openvino/", "coreml/", "tflite/")
_SKIP_EXT = (".bin", ".pth", ".pt", ".msgpack", ".h5", ".onnx", ".gguf", ".tflite")


class ModelNotFound(FileNotFoundError):
    pass


class DownloadError(RuntimeError):
    pass


# ----------------------------------------------------------------------------- resolve
def cache_root(cache_dir: Optional[str] = None) -> Path:
    if cache_dir:
        return Path(cache_dir)
    if os.environ.get("HF_HUB_CACHE"):
        return Path(os.environ["HF_HUB_CACHE"])
    home = os.environ.get("HF_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "huggingface")
    return Path(home) / "hub"


def repo_dir(root: Path, repo: str) -> Path:
    return Path(root) / ("models--" + repo.replace("/", "--"))


def _has_weights(d: Path) -> bool:
    return any(d.glob("*.safetensors")) or any(d.glob("*.gguf"))


def resolve_model_dir(model: str, cache_dir: Optional[str] = None, presets=()) -> str:
    """Preset name -> itself; directory with a config (or a .gguf file) -> itself; repository id ->
    its snapshot directory in the cache."""
    if model in presets:
        return model
    p = Path(model)
    if p.is_file() and p.suffix == ".gguf":
        return str(p)
    if p.is_dir() and ((p / "config.json").exists() or (p / "engine_config.json").exists() or any(p.glob("*.gguf"))):
        return str(p)
    root = cache_root(cache_dir)
    rd = repo_dir(root, model)
    hint = f"download it first:  metrale-b200 download {model}  (or: hf download {model})"
    if not rd.is_dir():
        raise ModelNotFound(f"model '{model}' is neither a preset, a checkpoint directory nor in the cache at {root}; {hint}")
    ref = rd / "refs" / "main"
    if not ref.exists():
        raise ModelNotFound(f"no default revision for '{model}': expected {ref}; the download may be incomplete; {hint}")
    rev = ref.read_text().strip()
    snap = rd / "snapshots" / rev
    if not snap.is_dir():
        raise ModelNotFound(f"refs/main of '{model}' points to '{rev}' but {snap} does not exist; {hint}")
    if not (snap / "config.json").exists() and not (snap / "params.json").exists():
        raise ModelNotFound(f"{snap} has no config.json / params.json: the download may be incomplete; {hint}")
    if not _has_weights(snap):
        raise ModelNotFound(f"{snap} has a config but no weight files: the download may be incomplete; {hint}")
    return str(snap)


def list_models(cache_dir: Optional[str] = None) -> List[dict]:
    """Repositories in the cache with their revision, size and completeness."""
    root = cache_root(cache_dir)
    out = []
    if not root.is_dir():
        return out
    for d in sorted(root.glob("models--*")):
        repo = d.name[len("models--"):].replace("--", "/")
        ref = d / "refs" / "main"
        rev = ref.read_text().strip() if ref.exists() else None
        snap = d / "snapshots" / rev if rev else None
        size = sum(f.stat().st_size for f in snap.rglob("*") if f.is_file()) if snap and snap.is_dir() else 0
        out.append({"repo": repo, "revision": rev, "bytes": size,
                    "complete": bool(snap and snap.is_dir() and (snap / "config.json").exists() and _has_weights(snap))})
    return out


# ----------------------------------------------------------------------------- download plan
@dataclass(frozen=True)
class RemoteFile:
    name: str
    size: Optional[int] = None


def is_contained(name: str) -> bool:
    if not name or name.startswith("/") or "\\" in name:
        return False
    if len(name) >= 2 and name[0].isalpha() and name[1] == ":":
        return False
    return all(c not in ("", ".", "..") for c in name.split("/"))


def is_weight(name: str) -> bool:
    return name.endswith(".safetensors") or name.endswith(".safetensors.index.json")


def wanted(name: str) -> bool:
    if not is_contained(name) or name.startswith(_SKIP_DIRS) or name.endswith(_SKIP_EXT):
        return False
    return is_weight(name) or ("/" not in name and name in METADATA)


def select(files: List[RemoteFile]) -> List[RemoteFile]:
    """Wanted files, metadata before weights and small before large (a broken repository fails fast)."""
    return sorted((f for f in files if wanted(f.name)), key=lambda f: (is_weight(f.name), f.size or 0, f.name))


# ----------------------------------------------------------------------------- fetch
def _open(url: str, token: Optional[str], start: int = 0, timeout: float = 30.0):
    headers = {"User-Agent": "metrale-b200"}
    if token:
        headers["Authorization"] = f"Bearer {token}"
    if start:
        headers["Range"] = f"bytes={start}-"
    return urllib.request.urlopen(urllib.request.Request(url, headers=headers), timeout=timeout)


def repo_info(endpoint: str, repo: str, revision: str = "main", token: Optional[str] = None) -> Tuple[str, List[RemoteFile]]:
    url = f"{endpoint.rstrip('/')}/api/models/{repo}/revision/{revision}?blobs=true"
    try:
        with _open(url, token) as r:
            info = json.loads(r.read())
    except urllib.error.HTTPError as e:
        raise DownloadError(f"{repo}@{revision}: HTTP {e.code} from {url}"
                            + (" (gated or private: set HF_TOKEN)" if e.code in (401, 403) else "")) from None
    except (urllib.error.URLError, OSError, ValueError) as e:
        raise DownloadError(f"{repo}@{revision}: cannot reach {endpoint}: {e}") from None
    files = [RemoteFile(s["rfilename"], s.get("size")) for s in info.get("siblings", []) if "rfilename" in s]
    return info.get("sha") or revision, files


def fetch_file(url: str, dest: Path, size: Optional[int], token: Optional[str] = None,
               progress: Optional[Callable[[int], None]] = None, cancelled: Optional[Callable[[], bool]] = None) -> None:
    """Downloads into ``<dest>.part`` (resuming what is there), renames when complete."""
    if dest.exists() and (size is None or dest.stat().st_size == size):
        return
    dest.parent.mkdir(parents=True, exist_ok=True)
    part = dest.with_name(dest.name + ".part")
    have = part.stat().st_size if part.exists() else 0
    if size is not None and have > size:
        part.unlink()
        have = 0
    if size is None or have < size:
        try:
            with _open(url, token, start=have) as r:
                if have and r.status != 206:           # the server ignored the Range header: start over
                    have = 0
                with open(part, "ab" if have else "wb") as f:
                    while True:
                        if cancelled is not None and cancelled():
                            raise DownloadError("cancelled")
                        chunk = r.read(1 << 20)
                        if not chunk:
                            break
                        f.write(chunk)
                        if progress is not None:
                            progress(len(chunk))
        except urllib.error.HTTPError as e:
            raise DownloadError(f"HTTP {e.code} for {url}") from None
        except (urllib.error.URLError, OSError) as e:
            raise DownloadError(f"{url}: {e}") from None
    got = part.stat().st_size
    if size is not None and got != size:
        raise DownloadError(f"{dest.name}: got {got} bytes, expected {size} (kept as {part.name} to resume)")
    os.replace(part, dest)


def download(repo: str, cache_dir: Optional[str] = None, endpoint: Optional[str] = None, revision: str = "main",
             token: Optional[str] = None, progress: Optional[Callable[[str, int, int], None]] = None,
             cancelled: Optional[Callable[[], bool]] = None) -> str:
    """Fetches `repo` into the cache and returns the snapshot directory."""
    endpoint = endpoint or os.environ.get("HF_ENDPOINT", "https://huggingface.co")
    token = token or os.environ.get("HF_TOKEN")
    root = cache_root(cache_dir)
    sha, files = repo_info(endpoint, repo, revision, token)
    plan = select(files)
    if not any(f.name.endswith(".safetensors") for f in plan):
        raise DownloadError(f"{repo}: no safetensors weights in the repository")
    if not is_contained(sha):
        raise DownloadError(f"{repo}: refusing revision name {sha!r}")
    snap = repo_dir(root, repo) / "snapshots" / sha
    snap.mkdir(parents=True, exist_ok=True)
    need = sum((f.size or 0) for f in plan
               if not ((snap / f.name).exists() and (snap / f.name).stat().st_size == (f.size or -1)))
    free = shutil.disk_usage(snap).free
    if need > free:
        raise DownloadError(f"{repo}: needs {need / 2**30:.1f} GiB, {free / 2**30:.1f} GiB free at {root}")
    total, done = sum(f.size or 0 for f in plan), 0
    for f in plan:
        def bump(n, _f=f):
            nonlocal done
            done += n
            if progress is not None:
                progress(_f.name, done, total)
        fetch_file(f"{endpoint.rstrip('/')}/{repo}/resolve/{sha}/{f.name}", snap / f.name, f.size, token, bump, cancelled)
    ref = repo_dir(root, repo) / "refs" / "main"
    ref.parent.mkdir(parents=True, exist_ok=True)
    tmp = ref.with_name("main.tmp")
    tmp.write_text(sha)
    os.replace(tmp, ref)                       # published last: resolve_model_dir never sees a partial snapshot
    return str(snap)
