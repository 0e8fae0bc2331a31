"""Model-hub registry service and its client.

The service keeps users, organisations, API keys, models, versions, files and metrics under one directory
(``db.json`` + ``blobs/``) and is served by the C++ HTTP front-end (``serving/native_http.py``); the client speaks
to it with ``urllib``. Verbs follow the reference hub (``model_hub/api/main.py:344-660``: models, versions,
upload / download, users, orgs, API keys, leaderboard; ``model_hub/api/client.py``; ``model_hub/hub.py:51-297``
module-level ``login / upload / download / search / list_models / leaderboard``).

Routes (JSON unless noted; write routes need ``Authorization: Bearer <token or API key>``):
  POST /api/users                      {username, password}            register
  POST /api/login                      {username, password}            -> {token}
  POST /api/keys                       {name}                          -> {key}        GET /api/keys   DELETE /api/keys/{name}
  POST /api/orgs                       {name}                          POST /api/orgs/{org}/members {username}
  GET  /api/models?q=&tag=             search                          POST /api/models {id, description, tags, private}
  GET  /api/models/{owner}/{name}      card + versions                 DELETE /api/models/{owner}/{name}
  POST /api/models/{owner}/{name}/versions {version, metrics}
  PUT  /api/models/{owner}/{name}/versions/{version}/files/{file}      raw bytes (upload)
  GET  /api/models/{owner}/{name}/versions/{version}/files/{file}      raw bytes (download)
  GET  /api/leaderboard?metric=&order=desc
"""
from __future__ import annotations

import hashlib
import json
import os
import secrets
import threading
import time
import urllib.error
import urllib.parse
import urllib.request
from typing import Dict, List, Optional

from ..security import crypto
from ..serving.native_http import HTTPError, NativeHttpServer


class HubRegistry:
    """State and rules of the hub, independent of the transport."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(os.path.join(root, "blobs"), exist_ok=True)
        self._path = os.path.join(root, "db.json")
        self._lock = threading.RLock()
        self.db = json.load(open(self._path)) if os.path.exists(self._path) else \
            {"users": {}, "orgs": {}, "models": {}, "tokens": {}, "keys": {}}

    def _save(self):
        tmp = self._path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.db, f)
        os.replace(tmp, self._path)

    # ---- identities
    def register(self, username: str, password: str):
        with self._lock:
            if not username or not username.replace("-", "").replace("_", "").isalnum():
                raise HTTPError(400, "username must be alphanumeric")
            if username in self.db["users"] or username in self.db["orgs"]:
                raise HTTPError(409, "name taken")
            if len(password) < 8:
                raise HTTPError(400, "password must have at least 8 characters")
            salt = secrets.token_bytes(16)
            self.db["users"][username] = {"salt": salt.hex(), "hash": crypto.pbkdf2_sha256(password.encode(), salt, 20000).hex(),
                                          "created": time.time()}
            self._save()

    def login(self, username: str, password: str) -> str:
        with self._lock:
            u = self.db["users"].get(username)
            ok = u is not None and crypto.ct_equal(bytes.fromhex(u["hash"]),
                                                   crypto.pbkdf2_sha256(password.encode(), bytes.fromhex(u["salt"]), 20000))
            if not ok:
                raise HTTPError(401, "bad credentials")
            tok = secrets.token_urlsafe(24)
            self.db["tokens"][hashlib.sha256(tok.encode()).hexdigest()] = {"user": username, "expires": time.time() + 86400}
            self._save()
            return tok

    def whoami(self, authorization: Optional[str]) -> str:
        if not authorization or not authorization.startswith("Bearer "):
            raise HTTPError(401, "bearer token or API key required")
        digest = hashlib.sha256(authorization[7:].encode()).hexdigest()
        with self._lock:
            t = self.db["tokens"].get(digest)
            if t and t["expires"] > time.time():
                return t["user"]
            k = self.db["keys"].get(digest)
            if k:
                return k["user"]
        raise HTTPError(401, "invalid or expired credentials")

    def create_key(self, user: str, name: str) -> str:
        with self._lock:
            key = "sxk_" + secrets.token_urlsafe(24)
            self.db["keys"][hashlib.sha256(key.encode()).hexdigest()] = {"user": user, "name": name, "created": time.time()}
            self._save()
            return key

    def list_keys(self, user: str) -> List[str]:
        return sorted(k["name"] for k in self.db["keys"].values() if k["user"] == user)

    def delete_key(self, user: str, name: str) -> bool:
        with self._lock:
            hit = [d for d, k in self.db["keys"].items() if k["user"] == user and k["name"] == name]
            for d in hit:
                del self.db["keys"][d]
            self._save()
            return bool(hit)

    def create_org(self, user: str, name: str):
        with self._lock:
            if name in self.db["orgs"] or name in self.db["users"]:
                raise HTTPError(409, "name taken")
            self.db["orgs"][name] = {"owner": user, "members": [user]}
            self._save()

    def add_member(self, user: str, org: str, member: str):
        with self._lock:
            o = self.db["orgs"].get(org)
            if o is None or member not in self.db["users"]:
                raise HTTPError(404, "unknown organisation or user")
            if o["owner"] != user:
                raise HTTPError(403, "only the owner adds members")
            if member not in o["members"]:
                o["members"].append(member)
            self._save()

    def _may_write(self, user: str, owner: str) -> bool:
        return user == owner or user in self.db["orgs"].get(owner, {}).get("members", [])

    # ---- models
    def create_model(self, user: str, model_id: str, description: str = "", tags=(), private: bool = False):
        owner, _, name = model_id.partition("/")
        with self._lock:
            if not name or not self._may_write(user, owner):
                raise HTTPError(403, "model id must be <your user or organisation>/<name>")
            if model_id in self.db["models"]:
                raise HTTPError(409, "model exists")
            self.db["models"][model_id] = {"description": description, "tags": list(tags), "private": bool(private),
                                           "created": time.time(), "downloads": 0, "versions": {}}
            self._save()

    def _model(self, model_id: str, user: Optional[str], write: bool = False) -> dict:
        m = self.db["models"].get(model_id)
        owner = model_id.split("/")[0]
        if m is None or (m["private"] and not (user and self._may_write(user, owner))):
            raise HTTPError(404, f"unknown model {model_id}")
        if write and not (user and self._may_write(user, owner)):
            raise HTTPError(403, "no write access")
        return m

    def add_version(self, user: str, model_id: str, version: str, metrics: Optional[Dict[str, float]] = None):
        with self._lock:
            m = self._model(model_id, user, write=True)
            if version in m["versions"]:
                raise HTTPError(409, "version exists")
            m["versions"][version] = {"metrics": metrics or {}, "files": {}, "created": time.time()}
            self._save()

    def put_file(self, user: str, model_id: str, version: str, name: str, data: bytes) -> str:
        with self._lock:
            m = self._model(model_id, user, write=True)
            v = m["versions"].get(version)
            if v is None:
                raise HTTPError(404, "unknown version")
            if "/" in name or name.startswith("."):
                raise HTTPError(400, "bad file name")
            digest = hashlib.sha256(data).hexdigest()
            with open(os.path.join(self.root, "blobs", digest), "wb") as f:  # content-addressed: equal files share a blob
                f.write(data)
            v["files"][name] = {"sha256": digest, "size": len(data)}
            self._save()
            return digest

    def get_file(self, user: Optional[str], model_id: str, version: str, name: str) -> bytes:
        with self._lock:
            m = self._model(model_id, user)
            f = m["versions"].get(version, {}).get("files", {}).get(name)
            if f is None:
                raise HTTPError(404, "unknown file")
            m["downloads"] += 1
            self._save()
        data = open(os.path.join(self.root, "blobs", f["sha256"]), "rb").read()
        if hashlib.sha256(data).hexdigest() != f["sha256"]:
            raise HTTPError(500, "stored blob is corrupt")
        return data

    def card(self, user: Optional[str], model_id: str) -> dict:
        m = self._model(model_id, user)
        return {"id": model_id, **{k: m[k] for k in ("description", "tags", "private", "downloads")},
                "versions": {v: {"metrics": i["metrics"], "files": i["files"]} for v, i in m["versions"].items()}}

    def delete_model(self, user: str, model_id: str):
        with self._lock:
            self._model(model_id, user, write=True)
            del self.db["models"][model_id]
            self._save()

    def search(self, user: Optional[str], q: str = "", tag: str = "") -> List[dict]:
        out = []
        for mid, m in sorted(self.db["models"].items()):
            if m["private"] and not (user and self._may_write(user, mid.split("/")[0])):
                continue
            if q.lower() in (mid + " " + m["description"]).lower() and (not tag or tag in m["tags"]):
                out.append({"id": mid, "tags": m["tags"], "downloads": m["downloads"], "versions": sorted(m["versions"])})
        return out

    def leaderboard(self, metric: str, descending: bool = True) -> List[dict]:
        rows = [{"id": mid, "version": v, metric: i["metrics"][metric]} for mid, m in self.db["models"].items() if not m["private"]
                for v, i in m["versions"].items() if metric in i["metrics"]]
        return sorted(rows, key=lambda r: r[metric], reverse=descending)


def serve_hub(root: str, port: int = 0, workers: int = 4, max_upload: int = 1 << 30) -> NativeHttpServer:
    """Starts the registry service; returns the running server (``.port``, ``.stop()``; ``.registry`` is its state)."""
    reg = HubRegistry(root)
    srv = NativeHttpServer(max_body=max_upload)
    srv.registry = reg

    def body_json(body):
        try:
            d = json.loads(body or b"{}")
        except ValueError:
            raise HTTPError(400, "body is not JSON")
        if not isinstance(d, dict):
            raise HTTPError(400, "body must be a JSON object")
        return d

    def user_of(p, required=True):
        if not required and "_authorization" not in p:
            return None
        return reg.whoami(p.get("_authorization"))

    def query(p):
        return {k: v[0] for k, v in urllib.parse.parse_qs(p.get("_query", "")).items()}

    mid = lambda p: f"{p['owner']}/{p['name']}"  # noqa: E731

    @srv.route("POST", "/api/users")
    def _(p, b):
        d = body_json(b)
        reg.register(str(d.get("username", "")), str(d.get("password", "")))
        return 201, {"username": d["username"]}

    @srv.route("POST", "/api/login")
    def _(p, b):
        d = body_json(b)
        return {"token": reg.login(str(d.get("username", "")), str(d.get("password", "")))}

    @srv.route("POST", "/api/keys")
    def _(p, b):
        return 201, {"key": reg.create_key(user_of(p), str(body_json(b).get("name", "default")))}

    @srv.route("GET", "/api/keys")
    def _(p, b):
        return {"keys": reg.list_keys(user_of(p))}

    @srv.route("DELETE", "/api/keys/{key_name}")
    def _(p, b):
        if not reg.delete_key(user_of(p), p["key_name"]):
            raise HTTPError(404, "unknown key")
        return {"deleted": p["key_name"]}

    @srv.route("POST", "/api/orgs")
    def _(p, b):
        reg.create_org(user_of(p), str(body_json(b).get("name", "")))
        return 201, {"ok": True}

    @srv.route("POST", "/api/orgs/{org}/members")
    def _(p, b):
        reg.add_member(user_of(p), p["org"], str(body_json(b).get("username", "")))
        return {"ok": True}

    @srv.route("GET", "/api/models")
    def _(p, b):
        q = query(p)
        return {"models": reg.search(user_of(p, required=False), q.get("q", ""), q.get("tag", ""))}

    @srv.route("POST", "/api/models")
    def _(p, b):
        d = body_json(b)
        reg.create_model(user_of(p), str(d.get("id", "")), str(d.get("description", "")), d.get("tags", []), bool(d.get("private")))
        return 201, {"id": d["id"]}

    @srv.route("GET", "/api/models/{owner}/{name}")
    def _(p, b):
        return reg.card(user_of(p, required=False), mid(p))

    @srv.route("DELETE", "/api/models/{owner}/{name}")
    def _(p, b):
        reg.delete_model(user_of(p), mid(p))
        return {"deleted": mid(p)}

    @srv.route("POST", "/api/models/{owner}/{name}/versions")
    def _(p, b):
        d = body_json(b)
        reg.add_version(user_of(p), mid(p), str(d.get("version", "")), d.get("metrics"))
        return 201, {"version": d.get("version")}

    @srv.route("PUT", "/api/models/{owner}/{name}/versions/{version}/files/{file}")
    def _(p, b):
        return 201, {"sha256": reg.put_file(user_of(p), mid(p), p["version"], p["file"], b)}

    @srv.route("GET", "/api/models/{owner}/{name}/versions/{version}/files/{file}")
    def _(p, b):
        return reg.get_file(user_of(p, required=False), mid(p), p["version"], p["file"])

    @srv.route("GET", "/api/leaderboard")
    def _(p, b):
        q = query(p)
        if "metric" not in q:
            raise HTTPError(400, "metric is required")
        return {"rows": reg.leaderboard(q["metric"], q.get("order", "desc") != "asc")}

    srv.start(port, workers)
    return srv


class HubClient:
    """HTTP client of the registry service (the reference's ``model_hub/api/client.py`` verbs)."""

    def __init__(self, url: str, token: Optional[str] = None):
        self.url, self.token = url.rstrip("/"), token

    def _call(self, method: str, path: str, body=None, raw: bool = False):
        data = body if isinstance(body, (bytes, type(None))) else json.dumps(body).encode()
        req = urllib.request.Request(self.url + path, data=data, method=method)
        if self.token:
            req.add_header("Authorization", f"Bearer {self.token}")
        try:
            with urllib.request.urlopen(req, timeout=60) as r:
                out = r.read()
        except urllib.error.HTTPError as e:
            msg = e.read().decode(errors="replace")
            try:
                msg = json.loads(msg).get("error", msg)
            except ValueError:
                pass
            raise RuntimeError(f"hub {method} {path}: {e.code} {msg}") from None
        return out if raw else json.loads(out)

    def register(self, username, password):
        return self._call("POST", "/api/users", {"username": username, "password": password})

    def login(self, username, password):
        self.token = self._call("POST", "/api/login", {"username": username, "password": password})["token"]
        return self.token

    def create_api_key(self, name="default"):
        return self._call("POST", "/api/keys", {"name": name})["key"]

    def list_api_keys(self):
        return self._call("GET", "/api/keys")["keys"]

    def delete_api_key(self, name):
        return self._call("DELETE", f"/api/keys/{name}")

    def create_org(self, name):
        return self._call("POST", "/api/orgs", {"name": name})

    def add_member(self, org, username):
        return self._call("POST", f"/api/orgs/{org}/members", {"username": username})

    def create_model(self, model_id, description="", tags=(), private=False):
        return self._call("POST", "/api/models", {"id": model_id, "description": description, "tags": list(tags), "private": private})

    def model_info(self, model_id):
        return self._call("GET", f"/api/models/{model_id}")

    def delete_model(self, model_id):
        return self._call("DELETE", f"/api/models/{model_id}")

    def search(self, q="", tag=""):
        return self._call("GET", "/api/models?" + urllib.parse.urlencode({"q": q, "tag": tag}))["models"]

    def list_models(self):
        return [m["id"] for m in self.search()]

    def leaderboard(self, metric, descending=True):
        return self._call("GET", "/api/leaderboard?" + urllib.parse.urlencode({"metric": metric, "order": "desc" if descending else "asc"}))["rows"]

    def upload(self, model_dir: str, model_id: str, version: str = "1.0.0", metrics: Optional[dict] = None):
        """Creates `version` and uploads every regular file of `model_dir`."""
        self._call("POST", f"/api/models/{model_id}/versions", {"version": version, "metrics": metrics or {}})
        sent = []
        for name in sorted(os.listdir(model_dir)):
            p = os.path.join(model_dir, name)
            if os.path.isfile(p):
                self._call("PUT", f"/api/models/{model_id}/versions/{version}/files/{urllib.parse.quote(name)}", open(p, "rb").read())
                sent.append(name)
        return sent

    def download(self, model_id: str, dest: str, version: Optional[str] = None) -> str:
        info = self.model_info(model_id)
        if not info["versions"]:
            raise RuntimeError(f"{model_id} has no versions")
        version = version or sorted(info["versions"])[-1]
        os.makedirs(dest, exist_ok=True)
        for name, meta in info["versions"][version]["files"].items():
            # file names come from the server: accept plain names only, never a path that could leave `dest`
            if (not name or os.path.basename(name) != name or name.startswith(".") or "\\" in name or "\x00" in name
                    or name in (os.curdir, os.pardir)):
                raise RuntimeError(f"registry sent an unsafe file name: {name!r}")
            data = self._call("GET", f"/api/models/{model_id}/versions/{version}/files/{urllib.parse.quote(name)}", raw=True)
            if hashlib.sha256(data).hexdigest() != meta["sha256"]:
                raise RuntimeError(f"checksum mismatch for {name}")
            with open(os.path.join(dest, name), "wb") as f:
                f.write(data)
        return dest

    def load(self, model_id: str, cache_dir: str, version: Optional[str] = None, **kw):
        from .model_hub import ModelHub
        return ModelHub.from_pretrained(self.download(model_id, os.path.join(cache_dir, model_id.replace("/", "__")), version), **kw)
