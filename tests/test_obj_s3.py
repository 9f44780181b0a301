"""The OBJ backend against an S3 service: `tests/fake_s3_server.py` keeps buckets in memory and checks the AWS
Signature Version 4 of every request with hashlib / hmac.  Covered: put, ranged get, head through `query_memory`,
keys with separators and characters that need escaping, a wrong secret, a missing key, multipart upload and ranged
download of a large object (`crtMinLimit`), virtual-hosted addressing, session tokens, unsigned payloads, connections the
server dropped while they were idle, and the service over TLS."""
import json
import os
import subprocess
import sys
import time
import urllib.request

import pytest
import torch

from nixl_b200 import nixl_agent, nixl_agent_config

HERE = os.path.dirname(os.path.abspath(__file__))
KEYS = {"access_key": "AKIDEXAMPLE", "secret_key": "wJalrXUtnFEMI/K7MDENG+bPxRfiCYEXAMPLEKEY"}


def _wait(agent, handle, seconds=60):
    deadline = time.time() + seconds
    state = agent.check_xfer_state(handle)
    while state == "PROC" and time.time() < deadline:
        state = agent.check_xfer_state(handle)
    return state


class _Server:
    def __init__(self, *flags, scheme="http"):
        self.proc = subprocess.Popen([sys.executable, os.path.join(HERE, "fake_s3_server.py"), "--bucket", "kv-cache", "--access-key", KEYS["access_key"],
                                      "--secret-key", KEYS["secret_key"], *flags], stdout=subprocess.PIPE, text=True)
        self.port = int(self.proc.stdout.readline())
        self.scheme = scheme
        self.endpoint = f"{scheme}://127.0.0.1:{self.port}"

    def admin(self, what):
        if self.scheme == "https":
            import ssl

            ctx = ssl.create_default_context()
            ctx.check_hostname = False
            ctx.verify_mode = ssl.CERT_NONE
            return json.loads(urllib.request.urlopen(f"{self.endpoint}/_admin/{what}", timeout=5, context=ctx).read())
        return json.loads(urllib.request.urlopen(f"{self.endpoint}/_admin/{what}", timeout=5).read())

    def params(self, **more):
        return dict(KEYS, bucket="kv-cache", endpoint_override=self.endpoint, **more)

    def close(self):
        self.proc.kill()
        self.proc.wait()


@pytest.fixture
def s3():
    server = _Server()
    yield server
    server.close()


def _roundtrip(agent, name, key, src, dev_id=1):
    """WRITE `src` to `key`, READ it back whole; returns the tensor read."""
    n = src.numel() * src.element_size()
    agent.register_memory([(0, n, dev_id, key)], "OBJ")
    remote = agent.get_xfer_descs([(0, n, dev_id)], "OBJ")
    h = agent.initialize_xfer("WRITE", agent.get_xfer_descs(src), remote, name)
    agent.transfer(h)
    assert _wait(agent, h) == "DONE"
    dst = torch.zeros_like(src)
    agent.register_memory(dst)
    h2 = agent.initialize_xfer("READ", agent.get_xfer_descs(dst), remote, name)
    agent.transfer(h2)
    assert _wait(agent, h2) == "DONE"
    agent.release_xfer_handle(h)
    agent.release_xfer_handle(h2)
    return dst


def test_put_get_head_and_ranges_with_signed_requests(s3):
    a = nixl_agent("s3_a", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", s3.params())
    src = torch.arange(1 << 16, dtype=torch.int32)
    a.register_memory(src)
    objs = [(0, src.numel() * 4, 1, "layers/0/kv block #1+a.bin")]  # separators and characters that must be escaped
    assert a.query_memory(objs, "OBJ", "OBJ")[0] is None
    assert torch.equal(_roundtrip(a, "s3_a", objs[0][3], src), src)
    info = a.query_memory(objs, "OBJ", "OBJ")[0]
    assert info is not None and int(info["size"]) == src.numel() * 4
    assert s3.admin("keys") == {"kv-cache": {"layers/0/kv block #1+a.bin": src.numel() * 4}}
    # a byte range out of the middle, into the middle of a tensor
    part = torch.zeros(1000, dtype=torch.int32)
    a.register_memory(part)
    h = a.initialize_xfer("READ", a.get_xfer_descs([(part.data_ptr() + 400, 2000, 0)], "DRAM"), a.get_xfer_descs([(12000, 2000, 1)], "OBJ"), "s3_a")
    a.transfer(h)
    assert _wait(a, h) == "DONE"
    assert torch.equal(part[100:600], src[3000:3500]) and int(part[:100].abs().sum()) == 0 and int(part[600:].abs().sum()) == 0
    # a range that runs past the end of the object is an error, not a short read (the registration, whose length is the
    # caller's claim, is larger than the object)
    a.register_memory([(0, src.numel() * 4 + 3000, 9, objs[0][3])], "OBJ")
    h = a.initialize_xfer("READ", a.get_xfer_descs([(part.data_ptr(), 4000, 0)], "DRAM"), a.get_xfer_descs([(src.numel() * 4 - 1000, 4000, 9)], "OBJ"), "s3_a")
    st = a.transfer(h)
    assert (st if st != "PROC" else _wait(a, h)) == "ERR"
    # writing at an offset is not something an object store does
    with pytest.raises(Exception):
        a.initialize_xfer("WRITE", a.get_xfer_descs([(part.data_ptr(), 4000, 0)], "DRAM"), a.get_xfer_descs([(4096, 4000, 1)], "OBJ"), "s3_a")
    stats = s3.admin("stats")
    assert stats["bad_signature"] == 0 and stats["unsigned_payload"] == 0
    assert stats["put"] == 1 and stats["get"] >= 3 and stats["head"] == 2
    assert stats["connections"] <= 10  # keep-alive: a handful of connections, not one per request


def test_a_missing_key_and_a_wrong_secret_are_told_apart(s3):
    a = nixl_agent("s3_b", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", s3.params())
    dst = torch.zeros(1024, dtype=torch.uint8)
    a.register_memory(dst)
    a.register_memory([(0, 1024, 1, "absent")], "OBJ")
    h = a.initialize_xfer("READ", a.get_xfer_descs(dst), a.get_xfer_descs([(0, 1024, 1)], "OBJ"), "s3_b")
    st = a.transfer(h)
    assert (st if st != "PROC" else _wait(a, h)) == "ERR"
    assert s3.admin("stats")["bad_signature"] == 0

    b = nixl_agent("s3_c", nixl_agent_config(backends=[]))
    b.create_backend("OBJ", s3.params(secret_key="not the secret"))
    src = torch.ones(1024, dtype=torch.uint8)
    b.register_memory(src)
    b.register_memory([(0, 1024, 1, "forbidden")], "OBJ")
    h = b.initialize_xfer("WRITE", b.get_xfer_descs(src), b.get_xfer_descs([(0, 1024, 1)], "OBJ"), "s3_c")
    st = b.transfer(h)
    assert (st if st != "PROC" else _wait(b, h)) == "ERR"
    assert s3.admin("stats")["bad_signature"] == 1
    assert s3.admin("keys") == {"kv-cache": {}}
    with pytest.raises(Exception):  # head is refused too, which is not the same as "no such key"
        b.query_memory([(0, 1024, 1, "forbidden")], "OBJ", "OBJ")


def test_large_objects_move_in_parts_side_by_side(s3):
    a = nixl_agent("s3_d", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", s3.params(crtMinLimit=str(5 << 20), num_threads="6"))
    src = torch.randint(0, 255, ((12 << 20) + 12345,), dtype=torch.uint8)
    small = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8)
    a.register_memory(src)
    a.register_memory(small)
    assert torch.equal(_roundtrip(a, "s3_d", "big.bin", src), src)
    assert torch.equal(_roundtrip(a, "s3_d", "small.bin", small, dev_id=2), small)
    stats = s3.admin("stats")
    assert stats["create_mpu"] == 1 and stats["part"] == 3 and stats["complete_mpu"] == 1 and stats["open_uploads"] == 0
    assert stats["put"] == 1            # the small one
    assert stats["get"] == 3 + 1        # three ranges of the large one, one request for the small one
    assert stats["bad_signature"] == 0
    assert s3.admin("keys")["kv-cache"] == {"big.bin": src.numel(), "small.bin": small.numel()}


def test_virtual_addressing_session_token_and_unsigned_payload():
    server = _Server("--session-token", "FwoGZXIvYXdzEXAMPLE")
    try:
        a = nixl_agent("s3_e", nixl_agent_config(backends=[]))
        a.create_backend("OBJ", server.params(use_virtual_addressing="true", session_token="FwoGZXIvYXdzEXAMPLE", payload_signing="false"))
        src = torch.arange(50000, dtype=torch.int16)
        a.register_memory(src)
        assert torch.equal(_roundtrip(a, "s3_e", "token.bin", src), src)
        stats = server.admin("stats")
        assert stats["bad_signature"] == 0 and stats["unsigned_payload"] == 1 and stats["virtual_host"] >= 2
        # without the token the same requests are refused
        b = nixl_agent("s3_f", nixl_agent_config(backends=[]))
        b.create_backend("OBJ", server.params())
        assert b.register_memory([(0, 16, 1, "token.bin")], "OBJ") is not None
        with pytest.raises(Exception):
            b.query_memory([(0, 16, 1, "token.bin")], "OBJ", "OBJ")
    finally:
        server.close()


def test_connections_the_server_dropped_while_idle_are_replaced():
    server = _Server("--close-after", "2")
    try:
        a = nixl_agent("s3_g", nixl_agent_config(backends=[]))
        a.create_backend("OBJ", server.params(num_threads="1"))
        src = torch.arange(4096, dtype=torch.int32)
        a.register_memory(src)
        for i in range(6):
            t = src + i
            a.register_memory(t)
            assert torch.equal(_roundtrip(a, "s3_g", f"k{i}", t, dev_id=i + 1), t)
        stats = server.admin("stats")
        assert stats["put"] == 6 and stats["get"] == 6 and stats["bad_signature"] == 0
        assert stats["connections"] >= 6  # twelve requests, two per connection
    finally:
        server.close()


def test_checksums_go_with_uploads_and_are_compared_on_downloads(s3):
    a = nixl_agent("s3_cs", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", s3.params(req_checksum="supported", resp_checksum="supported", crtMinLimit=str(5 << 20)))
    small = torch.randint(0, 255, (300000,), dtype=torch.uint8)
    big = torch.randint(0, 255, ((6 << 20) + 5,), dtype=torch.uint8)
    a.register_memory(small)
    a.register_memory(big)
    assert torch.equal(_roundtrip(a, "s3_cs", "sum-small.bin", small), small)
    assert torch.equal(_roundtrip(a, "s3_cs", "sum-big.bin", big, dev_id=2), big)
    stats = s3.admin("stats")
    assert stats["checksums_checked"] == 1 + 2 and stats["bad_checksum"] == 0  # one object, two parts
    assert stats["checksums_sent"] == 1  # the small one came back whole; ranges of the large one carry none
    assert stats["bad_signature"] == 0   # the checksum header is among the signed ones


def test_a_download_that_does_not_match_its_checksum_fails():
    server = _Server("--corrupt-downloads")
    try:
        a = nixl_agent("s3_cs2", nixl_agent_config(backends=[]))
        a.create_backend("OBJ", server.params(req_checksum="supported", resp_checksum="supported"))
        src = torch.arange(5000, dtype=torch.int32)
        dst = torch.zeros_like(src)
        a.register_memory(src)
        a.register_memory(dst)
        a.register_memory([(0, 20000, 1, "flipped.bin")], "OBJ")
        remote = a.get_xfer_descs([(0, 20000, 1)], "OBJ")
        h = a.initialize_xfer("WRITE", a.get_xfer_descs(src), remote, "s3_cs2")
        a.transfer(h)
        assert _wait(a, h) == "DONE"
        h = a.initialize_xfer("READ", a.get_xfer_descs(dst), remote, "s3_cs2")
        st = a.transfer(h)
        assert (st if st != "PROC" else _wait(a, h)) == "ERR"
        # without the comparison the flipped byte would have gone unnoticed
        b = nixl_agent("s3_cs3", nixl_agent_config(backends=[]))
        b.create_backend("OBJ", server.params())
        b.register_memory(dst)
        b.register_memory([(0, 20000, 1, "flipped.bin")], "OBJ")
        h = b.initialize_xfer("READ", b.get_xfer_descs(dst), b.get_xfer_descs([(0, 20000, 1)], "OBJ"), "s3_cs3")
        b.transfer(h)
        assert _wait(b, h) == "DONE"
    finally:
        server.close()


def test_a_service_that_says_slow_down_is_asked_again():
    server = _Server("--slow-down", "2")
    try:
        a = nixl_agent("s3_sd", nixl_agent_config(backends=[]))
        a.create_backend("OBJ", server.params(num_threads="1"))
        src = torch.arange(2000, dtype=torch.int32)
        a.register_memory(src)
        t0 = time.time()
        assert torch.equal(_roundtrip(a, "s3_sd", "patience.bin", src), src)  # the PUT is refused twice and goes through the third time
        assert time.time() - t0 >= 0.45  # 100 ms and 400 ms of waiting
        stats = server.admin("stats")
        assert stats["slow_downs"] == 2 and stats["put"] == 1 and stats["bad_signature"] == 0
    finally:
        server.close()
    # with one attempt only the refusal is the answer
    server = _Server("--slow-down", "1")
    try:
        b = nixl_agent("s3_sd2", nixl_agent_config(backends=[]))
        b.create_backend("OBJ", server.params(max_attempts="1"))
        src = torch.arange(100, dtype=torch.int32)
        b.register_memory(src)
        b.register_memory([(0, 400, 1, "impatient.bin")], "OBJ")
        h = b.initialize_xfer("WRITE", b.get_xfer_descs(src), b.get_xfer_descs([(0, 400, 1)], "OBJ"), "s3_sd2")
        st = b.transfer(h)
        assert (st if st != "PROC" else _wait(b, h)) == "ERR"
        assert server.admin("keys") == {"kv-cache": {}}
    finally:
        server.close()


def test_environment_variables_name_the_service(monkeypatch, s3):
    monkeypatch.setenv("AWS_ENDPOINT_OVERRIDE", s3.endpoint)
    monkeypatch.setenv("AWS_DEFAULT_BUCKET", "kv-cache")
    monkeypatch.setenv("AWS_ACCESS_KEY_ID", KEYS["access_key"])
    monkeypatch.setenv("AWS_SECRET_ACCESS_KEY", KEYS["secret_key"])
    a = nixl_agent("s3_h", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", {})
    src = torch.arange(1000, dtype=torch.float32)
    a.register_memory(src)
    assert torch.equal(_roundtrip(a, "s3_h", "env.bin", src), src)
    assert s3.admin("stats")["bad_signature"] == 0


def test_an_endpoint_that_does_not_answer_fails_the_request_not_the_process():
    a = nixl_agent("s3_i", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", dict(KEYS, bucket="kv-cache", endpoint_override="http://127.0.0.1:1", max_attempts="2"))
    src = torch.ones(64, dtype=torch.uint8)
    a.register_memory(src)
    a.register_memory([(0, 64, 1, "nowhere")], "OBJ")
    h = a.initialize_xfer("WRITE", a.get_xfer_descs(src), a.get_xfer_descs([(0, 64, 1)], "OBJ"), "s3_i")
    st = a.transfer(h)
    assert (st if st != "PROC" else _wait(a, h)) == "ERR"


def test_the_service_over_tls(tmp_path):
    try:
        import datetime

        from cryptography import x509
        from cryptography.hazmat.primitives import hashes, serialization
        from cryptography.hazmat.primitives.asymmetric import rsa
        from cryptography.x509.oid import NameOID
    except ImportError:
        pytest.skip("no library to make a certificate with")
    import ipaddress

    key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
    name = x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, "127.0.0.1")])
    now = datetime.datetime.now(datetime.timezone.utc)
    cert = (x509.CertificateBuilder().subject_name(name).issuer_name(name).public_key(key.public_key()).serial_number(x509.random_serial_number())
            .not_valid_before(now - datetime.timedelta(days=1)).not_valid_after(now + datetime.timedelta(days=2))
            .add_extension(x509.SubjectAlternativeName([x509.IPAddress(ipaddress.ip_address("127.0.0.1"))]), critical=False)
            .add_extension(x509.BasicConstraints(ca=True, path_length=None), critical=True).sign(key, hashes.SHA256()))
    cert_path, key_path = tmp_path / "cert.pem", tmp_path / "key.pem"
    cert_path.write_bytes(cert.public_bytes(serialization.Encoding.PEM))
    key_path.write_bytes(key.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.TraditionalOpenSSL, serialization.NoEncryption()))
    server = _Server("--tls", str(cert_path), str(key_path), scheme="https")
    try:
        a = nixl_agent("s3_j", nixl_agent_config(backends=[]))
        a.create_backend("OBJ", server.params(ca_bundle=str(cert_path)))
        src = torch.arange(1 << 15, dtype=torch.int32)
        a.register_memory(src)
        assert torch.equal(_roundtrip(a, "s3_j", "tls.bin", src), src)
        stats = server.admin("stats")
        assert stats["bad_signature"] == 0 and stats["unsigned_payload"] == 1  # over https the body is not hashed by default
        # a certificate nobody vouches for is refused
        b = nixl_agent("s3_k", nixl_agent_config(backends=[]))
        b.create_backend("OBJ", server.params())
        b.register_memory(src)
        b.register_memory([(0, 64, 1, "untrusted")], "OBJ")
        h = b.initialize_xfer("WRITE", b.get_xfer_descs([(src.data_ptr(), 64, 0)], "DRAM"), b.get_xfer_descs([(0, 64, 1)], "OBJ"), "s3_k")
        st = b.transfer(h)
        assert (st if st != "PROC" else _wait(b, h)) == "ERR"
        assert "untrusted" not in server.admin("keys")["kv-cache"]
    finally:
        server.close()


def test_nixlbench_against_the_service(s3):
    """The sweep tool with the object store as the far end: one object per block, put and got back; with the reference's
    flag spellings for the service's parameters."""
    exe = os.path.join(os.path.dirname(HERE), "nixl_b200", "bin", "nixlbench")
    env = dict(os.environ, NIXL_PLUGIN_DIR=os.path.join(os.path.dirname(HERE), "nixl_b200", "lib", "plugins"), NIXL_LOG_LEVEL="ERROR")
    common = ["--backend", "OBJ", "--mem", "DRAM", f"--obj_endpoint_override={s3.endpoint}", "--obj_bucket_name=kv-cache", f"--obj_access_key={KEYS['access_key']}",
              f"--obj_secret_key={KEYS['secret_key']}", "--min", "4096", "--max", "262144", "--batch", "3", "--iters", "6", "--warmup", "1", "--check"]
    for op in ("WRITE", "READ"):
        res = subprocess.run([exe, *common, "--op", op, "--obj-prefix", "bench-" + op.lower()], env=env, capture_output=True, text=True, timeout=180)
        assert res.returncode == 0, res.stdout + res.stderr
        rows = [l.split() for l in res.stdout.splitlines() if l and l[0].isdigit()]
        assert len(rows) == 7 and all(float(r[3]) > 0 for r in rows), res.stdout  # (the rate of 4 KiB objects may round to 0.00 GB/s)
    keys = s3.admin("keys")["kv-cache"]
    assert sorted(keys) == [f"bench-{op}-{i}" for op in ("read", "write") for i in range(3)] and set(keys.values()) == {262144}
    assert s3.admin("stats")["bad_signature"] == 0


def test_any_key_a_caller_may_think_of_round_trips(s3):
    """Keys drawn by hypothesis (spaces, punctuation that URLs reserve, other scripts, slashes): the path is escaped once
    on the wire and once more in the signature's view of it, and the service, which checks both, stores the key as given."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st

    a = nixl_agent("s3_keys", nixl_agent_config(backends=[]))
    a.create_backend("OBJ", s3.params())
    src = torch.arange(64, dtype=torch.uint8)
    dst = torch.zeros_like(src)
    a.register_memory(src)
    a.register_memory(dst)
    seen = []
    alphabet = st.one_of(st.characters(min_codepoint=0x20, max_codepoint=0x7E), st.sampled_from(list("äßçñ漢字ключ🙂")))

    @settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(st.text(alphabet, min_size=1, max_size=40).filter(lambda k: k.strip("/") == k and "//" not in k and k not in (".", "..") and "\\" not in k))
    def check(key):
        if key in seen:
            return
        seen.append(key)
        dev = len(seen)
        src.fill_(dev % 251)
        a.register_memory([(0, 64, dev, key)], "OBJ")
        remote = a.get_xfer_descs([(0, 64, dev)], "OBJ")
        for op, buf in (("WRITE", src), ("READ", dst)):
            h = a.initialize_xfer(op, a.get_xfer_descs(buf), remote, "s3_keys")
            a.transfer(h)
            assert _wait(a, h) == "DONE", key
            a.release_xfer_handle(h)
        assert torch.equal(src, dst), key

    check()
    stored = s3.admin("keys")["kv-cache"]
    assert sorted(stored) == sorted(seen) and s3.admin("stats")["bad_signature"] == 0


def test_the_infinia_name_reaches_an_s3_compatible_endpoint(s3):
    """INFINIA has no client of its own here; with an endpoint named it is the S3 client, `dataset` being the bucket."""
    import nixl_b200

    nixl_b200.add_plugin_directory(nixl_b200.STANDIN_PLUGIN_DIR)
    a = nixl_agent("s3_inf", nixl_agent_config(backends=[]))
    a.create_backend("INFINIA", dict(KEYS, dataset="kv-cache", endpoint_override=s3.endpoint, cluster="c", tenant="t"))
    src = torch.arange(2048, dtype=torch.int16)
    a.register_memory(src)
    assert torch.equal(_roundtrip(a, "s3_inf", "from-infinia-name.bin", src), src)
    assert "from-infinia-name.bin" in s3.admin("keys")["kv-cache"] and s3.admin("stats")["bad_signature"] == 0
