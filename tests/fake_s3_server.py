"""A stand-in S3 service for the OBJ backend's tests: buckets in memory, the REST calls the backend makes (PutObject,
ranged GetObject, HeadObject, DeleteObject, multipart upload), and a check of every request's AWS Signature Version 4
with hashlib / hmac, an implementation that shares nothing with the client's.  Runs as a process of its own:

    python fake_s3_server.py [--bucket NAME] [--access-key K --secret-key S] [--region R]
                             [--close-after N] [--tls CERT KEY] [--corrupt-downloads] [--slow-down N]

prints its port on the first line of stdout and serves until it is killed.  `--close-after N` drops every connection
after N requests without announcing it, which is what an idle keep-alive connection looks like to a client.
`GET /_admin/stats` answers with JSON counters; `GET /_admin/keys` with the keys of every bucket.
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
import zlib
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

MIN_PART = 5 << 20

STATE = {
    "buckets": {},      # bucket -> {key: bytes}
    "uploads": {},      # upload id -> {"bucket", "key", "parts": {n: bytes}}
    "stats": {"put": 0, "get": 0, "head": 0, "delete": 0, "create_mpu": 0, "part": 0, "complete_mpu": 0, "abort_mpu": 0,
              "bad_signature": 0, "unsigned_payload": 0, "connections": 0, "virtual_host": 0, "checksums_checked": 0, "checksums_sent": 0,
              "bad_checksum": 0, "slow_downs": 0},
    "slow_down": 0,     # this many of the next requests are answered with 503 SlowDown
    "lock": threading.Lock(),
    "next_upload": 1,
}
ARGS = None


def _hmac(key, msg):
    return hmac.new(key, msg.encode(), hashlib.sha256).digest()


def _crc(data):
    return base64.b64encode(zlib.crc32(data).to_bytes(4, "big")).decode()


def _bump(name):
    with STATE["lock"]:
        STATE["stats"][name] += 1


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    served = 0

    def log_message(self, *args):
        pass

    def setup(self):
        super().setup()
        self.request.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)  # headers and body leave as they are written
        _bump("connections")

    # ------------------------------------------------------------------ helpers
    def _reply(self, status, body=b"", headers=None, chunked=False):
        self.send_response(status)
        for k, v in (headers or {}).items():
            self.send_header(k, v)
        if chunked and body:
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()
            half = max(1, len(body) // 2)
            for piece in (body[:half], body[half:]):
                if piece:
                    self.wfile.write(b"%x\r\n%s\r\n" % (len(piece), piece))
            self.wfile.write(b"0\r\n\r\n")
        else:
            if self.command != "HEAD" or "Content-Length" not in (headers or {}):
                self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            if self.command != "HEAD":
                self.wfile.write(body)
        self.served += 1
        if ARGS.close_after and self.served >= ARGS.close_after:
            self.close_connection = True  # without saying so: the client finds out on its next request

    def _error(self, status, code, message):
        body = f"<?xml version='1.0'?><Error><Code>{code}</Code><Message>{message}</Message></Error>".encode()
        self._reply(status, body, {"Content-Type": "application/xml"}, chunked=True)

    def _split(self):
        """(bucket, key, query dict) of the request; virtual-hosted style when the Host header starts with a bucket."""
        parsed = urllib.parse.urlsplit(self.path)
        query = dict(urllib.parse.parse_qsl(parsed.query, keep_blank_values=True))
        path = urllib.parse.unquote(parsed.path)
        host = self.headers.get("Host", "")
        for b in STATE["buckets"]:
            if host.startswith(b + "."):
                _bump("virtual_host")
                return b, path.lstrip("/"), query
        parts = path.lstrip("/").split("/", 1)
        return parts[0], parts[1] if len(parts) > 1 else "", query

    def _check_signature(self, body):
        """True when the request carries a valid Signature Version 4 (or when the server runs without credentials)."""
        if not ARGS.access_key:
            return True
        auth = self.headers.get("Authorization", "")
        m = re.match(r"AWS4-HMAC-SHA256 Credential=([^/]+)/(\d{8})/([^/]+)/s3/aws4_request, SignedHeaders=([^,]+), Signature=([0-9a-f]{64})$", auth)
        if not m or m.group(1) != ARGS.access_key or m.group(3) != ARGS.region:
            return False
        date, signed, given = m.group(2), m.group(4).split(";"), m.group(5)
        amz_date = self.headers.get("x-amz-date", "")
        payload_hash = self.headers.get("x-amz-content-sha256", "")
        if not amz_date.startswith(date) or "host" not in signed or "x-amz-date" not in signed or "x-amz-content-sha256" not in signed:
            return False
        if ARGS.session_token and (self.headers.get("x-amz-security-token") != ARGS.session_token or "x-amz-security-token" not in signed):
            return False
        if payload_hash == "UNSIGNED-PAYLOAD":
            _bump("unsigned_payload")
        elif payload_hash != hashlib.sha256(body).hexdigest():
            return False
        parsed = urllib.parse.urlsplit(self.path)
        pairs = sorted((urllib.parse.quote(k, safe="-_.~"), urllib.parse.quote(v, safe="-_.~"))
                       for k, v in urllib.parse.parse_qsl(parsed.query, keep_blank_values=True))
        canonical_query = "&".join(f"{k}={v}" for k, v in pairs)
        canonical_uri = urllib.parse.quote(urllib.parse.unquote(parsed.path), safe="/-_.~")
        canonical_headers = "".join(f"{h}:{' '.join(self.headers.get(h, '').split())}\n" for h in signed)
        canonical = "\n".join([self.command, canonical_uri, canonical_query, canonical_headers, ";".join(signed), payload_hash])
        scope = f"{date}/{ARGS.region}/s3/aws4_request"
        to_sign = "\n".join(["AWS4-HMAC-SHA256", amz_date, scope, hashlib.sha256(canonical.encode()).hexdigest()])
        key = _hmac(_hmac(_hmac(_hmac(("AWS4" + ARGS.secret_key).encode(), date), ARGS.region), "s3"), "aws4_request")
        return hmac.compare_digest(hmac.new(key, to_sign.encode(), hashlib.sha256).hexdigest(), given)

    def _begin(self):
        """Reads the body, checks the signature and the bucket.  (bucket dict, key, query, body) or None after an error reply."""
        length = int(self.headers.get("Content-Length") or 0)
        body = self.rfile.read(length) if length else b""
        if self.path.startswith("/_admin/"):
            return None
        with STATE["lock"]:
            busy = STATE["slow_down"] > 0
            if busy:
                STATE["slow_down"] -= 1
                STATE["stats"]["slow_downs"] += 1
        if busy:
            self._error(503, "SlowDown", "Please reduce your request rate.")
            return None
        if not self._check_signature(body):
            _bump("bad_signature")
            self._error(403, "SignatureDoesNotMatch", "The request signature we calculated does not match the signature you provided.")
            return None
        bucket, key, query = self._split()
        if bucket not in STATE["buckets"]:
            self._error(404, "NoSuchBucket", "The specified bucket does not exist")
            return None
        return STATE["buckets"][bucket], key, query, body

    # ------------------------------------------------------------------ verbs
    def do_PUT(self):
        got = self._begin()
        if not got:
            return
        objects, key, query, body = got
        claimed = self.headers.get("x-amz-checksum-crc32")
        if claimed is not None:
            _bump("checksums_checked")
            if claimed != _crc(body) or "x-amz-checksum-crc32" not in self.headers.get("Authorization", "x-amz-checksum-crc32"):
                _bump("bad_checksum")
                return self._error(400, "BadDigest", "The CRC32 you specified did not match the calculated checksum.")
        if "partNumber" in query:
            _bump("part")
            up = STATE["uploads"].get(query.get("uploadId"))
            if not up or up["key"] != key:
                return self._error(404, "NoSuchUpload", "The specified upload does not exist")
            with STATE["lock"]:
                up["parts"][int(query["partNumber"])] = body
            return self._reply(200, b"", {"ETag": '"%s"' % hashlib.md5(body).hexdigest()})
        _bump("put")
        with STATE["lock"]:
            objects[key] = body
        self._reply(200, b"", {"ETag": '"%s"' % hashlib.md5(body).hexdigest()})

    def do_POST(self):
        got = self._begin()
        if not got:
            return
        objects, key, query, body = got
        if "uploads" in query:
            _bump("create_mpu")
            with STATE["lock"]:
                uid = "upload-%d" % STATE["next_upload"]
                STATE["next_upload"] += 1
                STATE["uploads"][uid] = {"key": key, "parts": {}}
            xml = f"<?xml version='1.0'?><InitiateMultipartUploadResult><Key>{key}</Key><UploadId>{uid}</UploadId></InitiateMultipartUploadResult>"
            return self._reply(200, xml.encode(), {"Content-Type": "application/xml"})
        if "uploadId" in query:
            _bump("complete_mpu")
            up = STATE["uploads"].get(query["uploadId"])
            if not up or up["key"] != key:
                return self._error(404, "NoSuchUpload", "The specified upload does not exist")
            listed = re.findall(r"<Part><PartNumber>(\d+)</PartNumber><ETag>([^<]*)</ETag></Part>", body.decode())
            numbers = [int(n) for n, _ in listed]
            if not listed or numbers != sorted(numbers) or numbers != list(range(1, len(numbers) + 1)):
                return self._error(400, "InvalidPartOrder", "The list of parts was not in ascending order")
            data = b""
            for i, (n, etag) in enumerate(listed):
                part = up["parts"].get(int(n))
                if part is None or etag.strip('"') != hashlib.md5(part).hexdigest():
                    return self._error(400, "InvalidPart", "One or more of the specified parts could not be found")
                if len(part) < MIN_PART and i != len(listed) - 1:
                    return self._error(400, "EntityTooSmall", "Your proposed upload is smaller than the minimum allowed size")
                data += part
            with STATE["lock"]:
                objects[key] = data
                del STATE["uploads"][query["uploadId"]]
            xml = f"<?xml version='1.0'?><CompleteMultipartUploadResult><Key>{key}</Key></CompleteMultipartUploadResult>"
            return self._reply(200, xml.encode(), {"Content-Type": "application/xml"})
        self._error(400, "InvalidRequest", "unsupported POST")

    def do_GET(self):
        if self.path == "/_admin/quit":  # for a parent that can only reach this process through its port
            self._reply(200, b"bye")
            threading.Thread(target=self.server.shutdown, daemon=True).start()
            return
        if self.path == "/_admin/stats":
            with STATE["lock"]:
                body = json.dumps(dict(STATE["stats"], open_uploads=len(STATE["uploads"]))).encode()
            return self._reply(200, body, {"Content-Type": "application/json"})
        if self.path == "/_admin/keys":
            with STATE["lock"]:
                body = json.dumps({b: {k: len(v) for k, v in objs.items()} for b, objs in STATE["buckets"].items()}).encode()
            return self._reply(200, body, {"Content-Type": "application/json"})
        got = self._begin()
        if not got:
            return
        objects, key, _, _ = got
        _bump("get")
        data = objects.get(key)
        if data is None:
            return self._error(404, "NoSuchKey", "The specified key does not exist.")
        rng = self.headers.get("Range")
        if not rng:
            return self._reply(200, data)
        m = re.match(r"bytes=(\d+)-(\d+)$", rng)
        if not m or int(m.group(1)) >= len(data):
            return self._error(416, "InvalidRange", "The requested range is not satisfiable")
        a, b = int(m.group(1)), min(int(m.group(2)), len(data) - 1)
        headers = {"Content-Range": f"bytes {a}-{b}/{len(data)}"}
        part = data[a:b + 1]
        if self.headers.get("x-amz-checksum-mode") == "ENABLED" and a == 0 and b == len(data) - 1:  # the whole object: its checksum goes along
            _bump("checksums_sent")
            headers["x-amz-checksum-crc32"] = _crc(data)
            if ARGS.corrupt_downloads and part:
                part = bytes([part[0] ^ 0xFF]) + part[1:]
        self._reply(206, part, headers)

    def do_HEAD(self):
        got = self._begin()
        if not got:
            return
        objects, key, _, _ = got
        _bump("head")
        data = objects.get(key)
        if data is None:
            return self._reply(404, b"")
        self._reply(200, b"", {"Content-Length": str(len(data)), "ETag": '"%s"' % hashlib.md5(data).hexdigest()})

    def do_DELETE(self):
        got = self._begin()
        if not got:
            return
        objects, key, query, _ = got
        if "uploadId" in query:
            _bump("abort_mpu")
            with STATE["lock"]:
                STATE["uploads"].pop(query["uploadId"], None)
            return self._reply(204, b"")
        _bump("delete")
        with STATE["lock"]:
            objects.pop(key, None)
        self._reply(204, b"")


def main():
    global ARGS
    ap = argparse.ArgumentParser()
    ap.add_argument("--bucket", action="append", default=[])
    ap.add_argument("--access-key", default="")
    ap.add_argument("--secret-key", default="")
    ap.add_argument("--session-token", default="")
    ap.add_argument("--region", default="us-east-1")
    ap.add_argument("--close-after", type=int, default=0)
    ap.add_argument("--slow-down", type=int, default=0, help="answer the first N requests with 503 SlowDown")
    ap.add_argument("--corrupt-downloads", action="store_true", help="flip a byte of every download that carries a checksum")
    ap.add_argument("--tls", nargs=2, metavar=("CERT", "KEY"))
    ARGS = ap.parse_args()
    STATE["slow_down"] = ARGS.slow_down
    for b in ARGS.bucket or ["test-bucket"]:
        STATE["buckets"][b] = {}
    server = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    server.daemon_threads = True
    if ARGS.tls:
        import ssl

        ctx = ssl.SSLContext(ssl.PROTOCOL_TLS_SERVER)
        ctx.load_cert_chain(ARGS.tls[0], ARGS.tls[1])
        server.socket = ctx.wrap_socket(server.socket, server_side=True)
    print(server.server_address[1], flush=True)
    server.serve_forever()


if __name__ == "__main__":
    sys.exit(main())
