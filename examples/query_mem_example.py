#!/usr/bin/env python
"""queryMem: ask a storage backend which files (or objects) exist before moving data.

The flow of the reference's examples/python/query_mem_example.py: descriptors name files in their
metadata string; the answer is one entry per descriptor, None for what does not exist."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nixl_b200 import nixl_agent, nixl_agent_config  # noqa: E402


def main():
    agent = nixl_agent("query_agent", nixl_agent_config(backends=[]))
    agent.create_backend("POSIX", {})
    with tempfile.TemporaryDirectory() as d:
        present = os.path.join(d, "present.bin")
        with open(present, "wb") as f:
            f.write(b"x" * 12345)
        files = [(0, 0, 0, present), (0, 0, 0, os.path.join(d, "absent.bin"))]
        for (_, _, _, path), info in zip(files, agent.query_memory(files, "POSIX", "FILE")):
            print(os.path.basename(path), "->", info)
        answers = agent.query_memory(files, "POSIX", "FILE")
        assert answers[0] is not None and answers[0]["size"] == "12345" and answers[1] is None

        # Object stores answer the same question by key.
        agent.create_backend("OBJ", {"bucket": d})
        objs = [(0, 0, 1, "present.bin"), (0, 0, 2, "no-such-key")]
        print("objects:", agent.query_memory(objs, "OBJ", "OBJ"))


if __name__ == "__main__":
    main()
