"""An in-process stand-in for etcd's JSON gateway (the /v3/... HTTP endpoints every etcd member serves), as far as the
native client uses it: kv put / range / deleterange / txn with a create-revision compare, leases with real expiry, token
authentication. Replies follow the gateway's conventions: 64-bit integers as strings, keys and values as base64, members
with default values left out, the keep-alive reply as a chunked stream of {"result": ...} lines."""
import base64
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


def _b(s):
    return base64.b64decode(s) if s else b""


def _e(b):
    return base64.b64encode(b).decode()


class FakeEtcd:
    def __init__(self, users=None, prefix="/v3"):
        self.kv = {}            # key bytes -> dict(value, lease, create, mod, version)
        self.leases = {}        # id -> dict(ttl, expire)
        self.rev = 1
        self.next_lease = 0x1000
        self.users = users or {}
        self.tokens = set()
        self.mu = threading.Lock()
        self.calls = []
        self.prefix = prefix
        self.down = False       # True: every call answers 503
        owner = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                raw = self.rfile.read(n) if n else b"{}"
                try:
                    body = json.loads(raw or b"{}")
                except ValueError:
                    return self._send(400, {"error": "bad json", "code": 3})
                path = self.path
                if not path.startswith(owner.prefix + "/"):
                    return self._send(404, {"error": "not found", "code": 5})
                op = path[len(owner.prefix):]
                if owner.down:
                    return self._send(503, {"error": "etcdserver: no leader", "code": 14})
                with owner.mu:
                    owner.calls.append(op)
                    if owner.users and op != "/auth/authenticate" and self.headers.get("Authorization") not in owner.tokens:
                        return self._send(401, {"error": "etcdserver: invalid auth token", "code": 16})
                    owner._expire()
                    status, reply = owner._handle(op, body)
                self._send(status, reply, chunked=(op == "/lease/keepalive"))

            def _send(self, status, obj, chunked=False):
                data = (json.dumps(obj) + ("\n" if chunked else "")).encode()
                self.send_response(status)
                self.send_header("Content-Type", "application/json")
                self.send_header("Connection", "close")
                if chunked:
                    self.send_header("Transfer-Encoding", "chunked")
                    self.end_headers()
                    self.wfile.write(b"%x\r\n%s\r\n0\r\n\r\n" % (len(data), data))
                else:
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                self.close_connection = True

        self.httpd = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)
        self.thread.start()

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()

    # ---- state (called with self.mu held) ----
    def _expire(self):
        now = time.monotonic()
        for lid in [i for i, l in self.leases.items() if l["expire"] <= now]:
            self._drop_lease(lid)

    def _drop_lease(self, lid):
        self.leases.pop(lid, None)
        for k in [k for k, e in self.kv.items() if e["lease"] == lid]:
            del self.kv[k]
            self.rev += 1

    def _header(self):
        return {"cluster_id": "1", "member_id": "1", "revision": str(self.rev), "raft_term": "2"}

    def _put(self, b):
        key, val, lease = _b(b.get("key")), _b(b.get("value")), int(b.get("lease", 0) or 0)
        if lease and lease not in self.leases:
            return 400, {"error": "etcdserver: requested lease not found", "code": 5}
        self.rev += 1
        old = self.kv.get(key)
        self.kv[key] = {"value": val, "lease": lease, "create": old["create"] if old else self.rev, "mod": self.rev,
                        "version": (old["version"] + 1) if old else 1}
        return 200, {"header": self._header()}

    def _select(self, b):
        key, end = _b(b.get("key")), _b(b.get("range_end"))
        if not end:
            return [key] if key in self.kv else []
        if end == b"\0":
            return sorted(k for k in self.kv if k >= key)
        return sorted(k for k in self.kv if key <= k < end)

    def _kvjson(self, k):
        e = self.kv[k]
        out = {"key": _e(k), "create_revision": str(e["create"]), "mod_revision": str(e["mod"]), "version": str(e["version"])}
        if e["value"]:
            out["value"] = _e(e["value"])
        if e["lease"]:
            out["lease"] = str(e["lease"])
        return out

    def _handle(self, op, b):
        if op == "/auth/authenticate":
            if self.users.get(b.get("name")) != b.get("password") or not self.users:
                return 400, {"error": "etcdserver: authentication failed, invalid user ID or password", "code": 3}
            tok = f"tok-{len(self.tokens)}-{time.monotonic_ns()}"
            self.tokens.add(tok)
            return 200, {"header": self._header(), "token": tok}
        if op == "/kv/put":
            return self._put(b)
        if op == "/kv/range":
            keys = self._select(b)
            out = {"header": self._header()}
            if keys:
                out["count"] = str(len(keys))
                if not b.get("count_only"):
                    out["kvs"] = [self._kvjson(k) for k in keys]
            return 200, out
        if op == "/kv/deleterange":
            keys = self._select(b)
            for k in keys:
                del self.kv[k]
            out = {"header": self._header()}
            if keys:
                self.rev += 1
                out["deleted"] = str(len(keys))
            return 200, out
        if op == "/kv/txn":
            ok = True
            for c in b.get("compare", []):
                if c.get("target") != "CREATE" or c.get("result") != "EQUAL":
                    return 400, {"error": "compare not supported by the stand-in", "code": 3}
                e = self.kv.get(_b(c.get("key")))
                ok = ok and (e["create"] if e else 0) == int(c.get("create_revision", 0) or 0)
            out = {"header": self._header()}
            if ok:
                out["succeeded"] = True
                out["responses"] = []
                for o in b.get("success", []):
                    st, r = self._put(o["request_put"])
                    if st != 200:
                        return st, r
                    out["responses"].append({"response_put": r})
            return 200, out
        if op == "/lease/grant":
            ttl = int(b.get("TTL", 0) or 0)
            if ttl <= 0:
                return 400, {"error": "etcdserver: bad TTL", "code": 3}
            self.next_lease += 1
            self.leases[self.next_lease] = {"ttl": ttl, "expire": time.monotonic() + ttl}
            return 200, {"header": self._header(), "ID": str(self.next_lease), "TTL": str(ttl)}
        if op == "/lease/keepalive":
            lid = int(b.get("ID", 0) or 0)
            l = self.leases.get(lid)
            res = {"header": self._header(), "ID": str(lid)}
            if l:
                l["expire"] = time.monotonic() + l["ttl"]
                res["TTL"] = str(l["ttl"])
            return 200, {"result": res}
        if op == "/lease/revoke":
            lid = int(b.get("ID", 0) or 0)
            if lid not in self.leases:
                return 404, {"error": "etcdserver: requested lease not found", "code": 5}
            self._drop_lease(lid)
            return 200, {"header": self._header()}
        return 404, {"error": "unknown call " + op, "code": 12}
