"""Random scatter lists against a model: two agents of one process, host memory, WRITE and READ requests whose pieces
are drawn by hypothesis (sizes from one byte to many chunks, pieces that touch, pieces in any order, the same request
posted twice); after every request both buffers must equal what numpy computes.  Run over the NVLINK backend (its
descriptor merging and host copy paths) and over the TCP backend with small chunks, so that requests are cut into many
messages, large pieces are split, and small ones share a message."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from nixl_b200 import nixl_agent, nixl_agent_config

SIZE = 1 << 18


@st.composite
def requests(draw):
    """(op, [(local offset, remote offset, length)]): local pieces never overlap each other, nor do remote pieces (a
    request that writes one place twice has no defined outcome)."""
    op = draw(st.sampled_from(["WRITE", "READ"]))
    n = draw(st.integers(1, 24))
    lengths = [draw(st.one_of(st.integers(1, 64), st.integers(65, 5000), st.integers(5001, 40000))) for _ in range(n)]
    total = sum(lengths)
    if total > SIZE:
        scale = SIZE / total / 1.01
        lengths = [max(1, int(x * scale)) for x in lengths]
        total = sum(lengths)
    slack = SIZE - total

    def layout(order_seed, gaps_seed):
        rng = np.random.default_rng(gaps_seed)
        cuts = np.sort(rng.integers(0, slack + 1, size=n)) if draw(st.booleans()) else np.zeros(n, dtype=np.int64)  # gaps, or all pieces touching
        order = np.random.default_rng(order_seed).permutation(n)
        offsets = [0] * n
        pos = 0
        prev_cut = 0
        for rank, idx in enumerate(order):
            pos += int(cuts[rank] - prev_cut)
            prev_cut = int(cuts[rank])
            offsets[idx] = pos
            pos += lengths[idx]
        return offsets

    lo = layout(draw(st.integers(0, 1 << 30)), draw(st.integers(0, 1 << 30)))
    ro = layout(draw(st.integers(0, 1 << 30)), draw(st.integers(0, 1 << 30)))
    return op, [(lo[i], ro[i], lengths[i]) for i in range(n)]


class _Pair:
    def __init__(self, backend, params, tag):
        self.a = nixl_agent(f"rnd_a_{tag}", nixl_agent_config(backends=[]))
        self.b = nixl_agent(f"rnd_b_{tag}", nixl_agent_config(backends=[]))
        self.a.create_backend(backend, params)
        self.b.create_backend(backend, params)
        self.src = torch.zeros(SIZE, dtype=torch.uint8)
        self.dst = torch.zeros(SIZE, dtype=torch.uint8)
        self.a.register_memory(self.src)
        self.b.register_memory(self.dst)
        self.a.add_remote_agent(self.b.get_agent_metadata())
        self.peer = f"rnd_b_{tag}"
        self.round = 0

    def run(self, op, pieces, twice):
        self.round += 1
        rng = np.random.default_rng(self.round)
        self.src.copy_(torch.from_numpy(rng.integers(0, 256, SIZE, dtype=np.uint8)))
        self.dst.copy_(torch.from_numpy(rng.integers(0, 256, SIZE, dtype=np.uint8)))
        model_src, model_dst = self.src.numpy().copy(), self.dst.numpy().copy()
        for lo, ro, n in pieces:
            if op == "WRITE":
                model_dst[ro:ro + n] = model_src[lo:lo + n]
            else:
                model_src[lo:lo + n] = model_dst[ro:ro + n]
        p, q = self.src.data_ptr(), self.dst.data_ptr()
        local = self.a.get_xfer_descs([(p + lo, n, 0) for lo, _, n in pieces], "DRAM")
        remote = self.a.get_xfer_descs([(q + ro, n, 0) for _, ro, n in pieces], "DRAM")
        h = self.a.initialize_xfer(op, local, remote, self.peer)
        for _ in range(2 if twice else 1):
            state = self.a.transfer(h)
            while state == "PROC":
                state = self.a.check_xfer_state(h)
            assert state == "DONE"
        self.a.release_xfer_handle(h)
        assert np.array_equal(self.src.numpy(), model_src), (op, pieces)
        assert np.array_equal(self.dst.numpy(), model_dst), (op, pieces)


_pairs = {}


def _pair(backend):
    if backend not in _pairs:
        params = {"address": "127.0.0.1", "rails": "3", "chunk_bytes": "4096"} if backend == "TCP" else {}
        _pairs[backend] = _Pair(backend, params, backend.lower())
    return _pairs[backend]


@pytest.mark.parametrize("backend", ["NVLINK", "TCP"])
def test_random_requests_leave_both_buffers_as_the_model_says(backend):
    pair = _pair(backend)

    @settings(max_examples=150, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(requests(), st.booleans())
    def check(request, twice):
        pair.run(request[0], request[1], twice)

    check()


@pytest.mark.parametrize("queue", ["", "use_aio", "use_uring", "use_posix_aio"])
def test_random_file_requests_against_a_model(tmp_path, queue):
    """The same drawing of pieces between host memory and a file, through every queue implementation of the POSIX
    backend: after a WRITE the file holds what numpy says, after a READ the buffer does."""
    import os

    agent = nixl_agent(f"rnd_file_{queue or 'pool'}", nixl_agent_config(backends=[]))
    try:
        agent.create_backend("POSIX", {queue: "true"} if queue else {})
    except Exception:
        pytest.skip(f"{queue} is not available on this kernel")
    buf = torch.zeros(SIZE, dtype=torch.uint8)
    agent.register_memory(buf)
    path = tmp_path / "blocks.bin"
    fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o644)
    os.ftruncate(fd, SIZE)
    agent.register_memory([(0, SIZE, fd, "")], "FILE")
    model_file = np.zeros(SIZE, dtype=np.uint8)
    counter = [0]

    @settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(requests())
    def check(request):
        op, pieces = request
        counter[0] += 1
        buf.copy_(torch.from_numpy(np.random.default_rng(counter[0]).integers(0, 256, SIZE, dtype=np.uint8)))
        model_buf = buf.numpy().copy()
        for lo, ro, n in pieces:
            if op == "WRITE":
                model_file[ro:ro + n] = model_buf[lo:lo + n]
            else:
                model_buf[lo:lo + n] = model_file[ro:ro + n]
        p = buf.data_ptr()
        h = agent.initialize_xfer(op, agent.get_xfer_descs([(p + lo, n, 0) for lo, _, n in pieces], "DRAM"),
                                  agent.get_xfer_descs([(ro, n, fd) for _, ro, n in pieces], "FILE"), agent.name)
        state = agent.transfer(h)
        while state == "PROC":
            state = agent.check_xfer_state(h)
        assert state == "DONE"
        agent.release_xfer_handle(h)
        assert np.array_equal(buf.numpy(), model_buf)
        assert np.array_equal(np.fromfile(path, dtype=np.uint8), model_file)

    try:
        check()
    finally:
        os.close(fd)
