"""A stand-in for etcd's v3 JSON gateway (put / range / deleterange over a dict) for the metadata tests.
Prints its port on the first line of stdout and serves until terminated; GET /keys lists the stored keys."""
import base64
import json
import sys
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

KV = {}
LOCK = threading.Lock()


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, *a):
        pass

    def _reply(self, obj):
        data = json.dumps(obj).encode()
        self.send_response(200)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.send_header("Connection", "close")
        self.end_headers()
        self.wfile.write(data)

    def do_GET(self):
        with LOCK:
            self._reply(sorted(KV))

    def do_POST(self):
        body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", "0"))) or b"{}")
        key = base64.b64decode(body.get("key", "")).decode()
        with LOCK:
            if self.path == "/v3/kv/put":
                KV[key] = base64.b64decode(body.get("value", ""))
                reply = {"header": {"revision": "1"}}
            elif self.path == "/v3/kv/range":
                reply = {"header": {"revision": "1"}}
                if key in KV:
                    reply["kvs"] = [{"key": body["key"], "value": base64.b64encode(KV[key]).decode()}]
                    reply["count"] = "1"
            elif self.path == "/v3/kv/deleterange":
                reply = {"header": {"revision": "1"}, "deleted": "1" if KV.pop(key, None) is not None else "0"}
            else:
                self.send_error(404)
                return
        self._reply(reply)


if __name__ == "__main__":
    server = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    print(server.server_address[1], flush=True)
    server.serve_forever()
