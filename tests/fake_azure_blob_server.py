"""A stand-in for Azure Blob Storage (in the shape of the storage emulator: the account is the first piece of the path)
for the AZURE_BLOB backend's tests: Put Blob, ranged Get Blob, Get Blob Properties, Delete Blob, Put Block and Put Block
List, every request checked against the account's Shared Key with hashlib / hmac / base64, an implementation that shares
nothing with the client's.  Runs as a process of its own:

    python fake_azure_blob_server.py [--account NAME] [--key BASE64] [--container NAME] [--sas TEXT]

prints its port on the first line of stdout.  `GET /_admin/stats` and `GET /_admin/blobs` answer with JSON.
With `--sas TEXT` requests are accepted when their query string carries `sig=TEXT` instead of a Shared Key.
"""
import argparse
import base64
import hashlib
import hmac
import json
import re
import socket
import sys
import threading
import urllib.parse
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

STATE = {
    "blobs": {},    # container -> {name: bytes}
    "blocks": {},   # (container, name) -> {block id: bytes}
    "stats": {"put_blob": 0, "get_blob": 0, "head": 0, "delete": 0, "put_block": 0, "put_block_list": 0, "bad_signature": 0, "sas": 0},
    "lock": threading.Lock(),
}
ARGS = None


def _bump(name):
    with STATE["lock"]:
        STATE["stats"][name] += 1


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, *args):
        pass

    def setup(self):
        super().setup()
        self.request.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)  # headers and body leave as they are written

    def _reply(self, status, body=b"", headers=None):
        self.send_response(status)
        for k, v in (headers or {}).items():
            self.send_header(k, v)
        if "Content-Length" not in (headers or {}):
            self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        if self.command != "HEAD":
            self.wfile.write(body)

    def _error(self, status, code, message):
        self._reply(status, f"<?xml version='1.0'?><Error><Code>{code}</Code><Message>{message}</Message></Error>".encode(),
                    {"Content-Type": "application/xml", "x-ms-error-code": code})

    def _authorised(self, length):
        parsed = urllib.parse.urlsplit(self.path)
        query = urllib.parse.parse_qsl(parsed.query, keep_blank_values=True)
        if ARGS.sas:
            if dict(query).get("sig") == ARGS.sas:
                _bump("sas")
                return True
            return False
        auth = self.headers.get("Authorization", "")
        m = re.match(r"SharedKey ([^:]+):(.+)$", auth)
        if not m or m.group(1) != ARGS.account:
            return False
        h = lambda name: self.headers.get(name, "")  # noqa: E731
        ms = sorted((k.lower(), " ".join(v.split())) for k, v in self.headers.items() if k.lower().startswith("x-ms-"))
        if not any(k == "x-ms-date" for k, _ in ms) or not any(k == "x-ms-version" for k, _ in ms):
            return False
        resource = "/" + ARGS.account + parsed.path
        for k, v in sorted((k.lower(), v) for k, v in query):
            resource += f"\n{k}:{v}"
        text = "\n".join([self.command, h("Content-Encoding"), h("Content-Language"), str(length) if length else "", h("Content-MD5"), h("Content-Type"),
                          h("Date"), h("If-Modified-Since"), h("If-Match"), h("If-None-Match"), h("If-Unmodified-Since"), h("Range")]) + "\n"
        text += "".join(f"{k}:{v}\n" for k, v in ms) + resource
        want = base64.b64encode(hmac.new(base64.b64decode(ARGS.key), text.encode(), hashlib.sha256).digest()).decode()
        return hmac.compare_digest(want, m.group(2))

    def _begin(self):
        length = int(self.headers.get("Content-Length") or 0)
        body = self.rfile.read(length) if length else b""
        if self.path.startswith("/_admin/"):
            return None
        if not self._authorised(length):
            _bump("bad_signature")
            self._error(403, "AuthenticationFailed", "Server failed to authenticate the request.")
            return None
        parsed = urllib.parse.urlsplit(self.path)
        pieces = urllib.parse.unquote(parsed.path).lstrip("/").split("/", 2)
        if len(pieces) < 3 or pieces[0] != ARGS.account:
            self._error(400, "InvalidUri", "The requested URI does not represent any resource on the server.")
            return None
        if pieces[1] not in STATE["blobs"]:
            self._error(404, "ContainerNotFound", "The specified container does not exist.")
            return None
        return pieces[1], pieces[2], dict(urllib.parse.parse_qsl(parsed.query, keep_blank_values=True)), body

    def do_PUT(self):
        got = self._begin()
        if not got:
            return
        container, name, query, body = got
        if query.get("comp") == "block":
            _bump("put_block")
            with STATE["lock"]:
                STATE["blocks"].setdefault((container, name), {})[query.get("blockid", "")] = body
            return self._reply(201)
        if query.get("comp") == "blocklist":
            _bump("put_block_list")
            ids = re.findall(r"<Latest>([^<]*)</Latest>", body.decode())
            staged = STATE["blocks"].get((container, name), {})
            if not ids or any(i not in staged for i in ids) or len({len(i) for i in ids}) != 1:
                return self._error(400, "InvalidBlockList", "The specified block list is invalid.")
            with STATE["lock"]:
                STATE["blobs"][container][name] = b"".join(staged[i] for i in ids)
                STATE["blocks"].pop((container, name), None)
            return self._reply(201)
        if self.headers.get("x-ms-blob-type") != "BlockBlob":
            return self._error(400, "MissingRequiredHeader", "x-ms-blob-type")
        _bump("put_blob")
        with STATE["lock"]:
            STATE["blobs"][container][name] = body
        self._reply(201, b"", {"ETag": '"%s"' % hashlib.md5(body).hexdigest()})

    def do_GET(self):
        if self.path == "/_admin/quit":  # for a parent that can only reach this process through its port
            self._reply(200, b"bye")
            threading.Thread(target=self.server.shutdown, daemon=True).start()
            return
        if self.path == "/_admin/stats":
            with STATE["lock"]:
                return self._reply(200, json.dumps(dict(STATE["stats"], staged=len(STATE["blocks"]))).encode())
        if self.path == "/_admin/blobs":
            with STATE["lock"]:
                return self._reply(200, json.dumps({c: {k: len(v) for k, v in b.items()} for c, b in STATE["blobs"].items()}).encode())
        got = self._begin()
        if not got:
            return
        container, name, _, _ = got
        _bump("get_blob")
        data = STATE["blobs"][container].get(name)
        if data is None:
            return self._error(404, "BlobNotFound", "The specified blob does not exist.")
        rng = self.headers.get("x-ms-range") or self.headers.get("Range")
        if not rng:
            return self._reply(200, data)
        m = re.match(r"bytes=(\d+)-(\d+)$", rng)
        if not m or int(m.group(1)) >= len(data):
            return self._error(416, "InvalidRange", "The range specified is invalid for the current size of the resource.")
        a, b = int(m.group(1)), min(int(m.group(2)), len(data) - 1)
        self._reply(206, data[a:b + 1], {"Content-Range": f"bytes {a}-{b}/{len(data)}"})

    def do_HEAD(self):
        got = self._begin()
        if not got:
            return
        container, name, _, _ = got
        _bump("head")
        data = STATE["blobs"][container].get(name)
        if data is None:
            return self._reply(404, b"")
        self._reply(200, b"", {"Content-Length": str(len(data)), "x-ms-blob-type": "BlockBlob"})

    def do_DELETE(self):
        got = self._begin()
        if not got:
            return
        container, name, _, _ = got
        _bump("delete")
        with STATE["lock"]:
            STATE["blobs"][container].pop(name, None)
        self._reply(202)


def main():
    global ARGS
    ap = argparse.ArgumentParser()
    ap.add_argument("--account", default="devstoreaccount1")
    ap.add_argument("--key", default=base64.b64encode(b"not a secret, a test key of some length").decode())
    ap.add_argument("--container", action="append", default=[])
    ap.add_argument("--sas", default="")
    ARGS = ap.parse_args()
    for c in ARGS.container or ["kv-cache"]:
        STATE["blobs"][c] = {}
    server = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    server.daemon_threads = True
    print(server.server_address[1], flush=True)
    server.serve_forever()


if __name__ == "__main__":
    sys.exit(main())
