#!/usr/bin/env python
"""Reads the telemetry ring that an agent with ``NIXL_TELEMETRY_ENABLE=1`` and
``NIXL_TELEMETRY_DIR=<dir>`` writes to ``<dir>/<agent name>`` (BUFFER exporter) and prints the
events.  Counterpart of the reference's examples/python/telemetry_reader.py; the ring layout is
documented in csrc/src/core/telemetry/ring_file.h."""
import mmap
import struct
import sys
import time

EVENT_NAMES = [
    "agent_tx_bytes", "agent_rx_bytes", "agent_tx_requests_num", "agent_rx_requests_num", "agent_memory_registered",
    "agent_memory_deregistered", "agent_xfer_time", "agent_xfer_post_time", "agent_err_not_posted", "agent_err_invalid_param",
    "agent_err_backend", "agent_err_not_found", "agent_err_mismatch", "agent_err_not_allowed", "agent_err_repost_active",
    "agent_err_unknown", "agent_err_not_supported", "agent_err_remote_disconnect", "agent_err_canceled", "agent_err_no_telemetry",
    "agent_telemetry_events_dropped",
]
HEADER = struct.Struct("<IIIIQQQ24x")  # magic, version, record size, capacity, head, tail, dropped
RECORD = struct.Struct("<QI4xQ")       # timestamp us, event type, value


def drain(path, follow=False):
    with open(path, "r+b") as f:
        m = mmap.mmap(f.fileno(), 0)
        magic, version, rec_size, capacity, _, _, _ = HEADER.unpack_from(m, 0)
        if magic != 0x4E585242:
            raise SystemExit(f"{path} is not a telemetry ring")
        print(f"# format version {version}, {capacity} slots of {rec_size} bytes")
        while True:
            _, _, _, _, head, tail, dropped = HEADER.unpack_from(m, 0)
            while tail < head:
                ts, kind, value = RECORD.unpack_from(m, HEADER.size + (tail % capacity) * rec_size)
                name = EVENT_NAMES[kind] if kind < len(EVENT_NAMES) else f"event_{kind}"
                print(f"{ts / 1e6:.6f} {name} {value}")
                tail += 1
                struct.pack_into("<Q", m, 24, tail)  # consume: advance the tail word
            if not follow:
                if dropped:
                    print(f"# {dropped} events were dropped because the ring was full")
                return
            time.sleep(0.1)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: telemetry_reader.py <NIXL_TELEMETRY_DIR>/<agent> [--follow]")
    drain(sys.argv[1], "--follow" in sys.argv)
