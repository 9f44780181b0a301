"""A stand-in for etcd's v3 JSON gateway (put / range / deleterange over a dict, and a watch stream) for the
metadata tests.  Prints its port on the first line of stdout and serves until terminated; GET /keys lists the
stored keys, GET /watchers the number of open watch streams.  With ``--no-watch`` POST /v3/watch answers 404, as a
gateway without that endpoint would."""
import base64
import json
import queue
import sys
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

KV = {}
LOCK = threading.Lock()
WATCHERS = []  # (prefix start, prefix end, queue) of every open watch stream
NO_WATCH = "--no-watch" in sys.argv


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
            self._reply(len(WATCHERS) if self.path == "/watchers" else sorted(KV))

    def _watch(self, body):
        """Streams one JSON object per line, chunked: first the creation notice, then a line per event."""
        if NO_WATCH:
            self.send_error(404)
            return
        req = body.get("create_request", {})
        start = base64.b64decode(req.get("key", "")).decode()
        end = base64.b64decode(req.get("range_end", "")).decode()
        q = queue.Queue()
        entry = (start, end, q)
        with LOCK:
            WATCHERS.append(entry)
        self.send_response(200)
        self.send_header("Content-Type", "application/json")
        self.send_header("Transfer-Encoding", "chunked")
        self.end_headers()

        def chunk(obj):
            data = (json.dumps(obj) + "\n").encode()
            self.wfile.write(b"%x\r\n" % len(data) + data + b"\r\n")
            self.wfile.flush()

        try:
            chunk({"result": {"header": {"revision": "1"}, "created": True}})
            while True:
                try:
                    event = q.get(timeout=0.5)
                except queue.Empty:
                    chunk({"result": {"header": {"revision": "1"}}})  # progress notice: also finds a closed connection
                    continue
                chunk({"result": {"header": {"revision": "2"}, "events": [event]}})
        except (BrokenPipeError, ConnectionResetError, OSError):
            pass
        finally:
            with LOCK:
                WATCHERS.remove(entry)

    def do_POST(self):
        body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", "0"))) or b"{}")
        if self.path == "/v3/watch":
            self._watch(body)
            return
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
                gone = KV.pop(key, None) is not None
                reply = {"header": {"revision": "1"}, "deleted": "1" if gone else "0"}
                if gone:  # proto3 JSON: PUT is the default type and is omitted, DELETE is spelled out
                    for start, end, q in WATCHERS:
                        if start <= key < end:
                            q.put({"type": "DELETE", "kv": {"key": body["key"], "mod_revision": "2"}})
            else:
                self.send_error(404)
                return
        self._reply(reply)


if __name__ == "__main__":
    server = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    print(server.server_address[1], flush=True)
    server.serve_forever()
