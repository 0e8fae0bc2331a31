"""Model hub: presets, from_pretrained, weight formats, local registry."""
from .formats import (load_hub_container, load_npz, load_safetensors, save_hub_container, save_npz,  # noqa: F401
                      save_safetensors)
from .model_hub import (HF_WEIGHT_MAP, Hub, ModelHub, convert_hf_to_sneppx, from_pretrained, map_hf_name,  # noqa: F401
                        reference_tensor_order)

# Module-level verbs of the reference's hub facade (model_hub/hub.py:51-297): they act on the default local hub, or on a
# registry service after ``login(url, user, password)``.
_session = {"client": None, "hub": None}


def _local():
    if _session["hub"] is None:
        _session["hub"] = Hub()
    return _session["hub"]


def login(url: str, username: str, password: str):
    from .registry_server import HubClient
    c = HubClient(url)
    c.login(username, password)
    _session["client"] = c
    return c


def logout():
    _session["client"] = None


def list_models():
    return _session["client"].list_models() if _session["client"] else _local().list_models()


def search(query: str = "", tag=None):
    return _session["client"].search(query, tag or "") if _session["client"] else _local().search(query, tag)


def upload(model_dir: str, model_id: str, version: str = "1.0.0", **kw):
    if _session["client"]:
        return _session["client"].upload(model_dir, model_id, version, kw.get("metrics"))
    return _local().upload(model_dir, model_id, version, kw.get("tags", ()), kw.get("metrics"))


def download(model_id: str, version=None, dest=None):
    if _session["client"]:
        import os
        return _session["client"].download(model_id, dest or os.path.join(os.path.expanduser("~/.sneppx/cache"), model_id.replace("/", "__")), version)
    return _local().download(model_id, version)


def load(model_id: str, version=None, **kw):
    return ModelHub.from_pretrained(download(model_id, version), **kw)


def leaderboard(metric: str, higher_is_better: bool = True):
    return _session["client"].leaderboard(metric, higher_is_better) if _session["client"] else _local().leaderboard(metric, higher_is_better)
