"""Hand-encoding of VMProgram v3 blobs with `struct`, independent of the
reference's Python package (so it runs anywhere).  Same role as the `Builder`
in the reference's device test (pjrt_plugin/src/runtime_test.cc:20-104): no
tensor instructions, only the schedule sections the device executes.
"""
from __future__ import annotations

import struct

NOP, BARRIER, WHILE, IF, FOR = 0xFFFFFFFF, 0xFFFFFFFE, 0xFFFFFFFD, 0xFFFFFFFC, 0xFFFFFFFB
FLAG_NONE = 0xFFFFFFFF
DT_SIZE = {0: 4, 1: 4, 2: 4, 3: 1, 4: 8, 5: 8, 6: 2, 7: 2}


class Builder:
    def __init__(self, n_lanes: int):
        self.n_lanes = n_lanes
        self.bufs = []           # (offset, size, dtype)
        self.arena = 0
        self.inputs, self.outputs = [], []
        self.in_dims, self.out_dims = [], []
        self.consts = []         # (buffer id, bytes)
        self.aux = []
        self.tasks = []          # 12-tuples
        self.lanes = [[] for _ in range(n_lanes)]
        self.root_lens = [0] * n_lanes

    def buf(self, elems: int, dtype: int = 0) -> int:
        size = elems * DT_SIZE[dtype]
        self.bufs.append((self.arena, size, dtype))
        self.arena = (self.arena + size + 63) & ~63
        return len(self.bufs) - 1

    def task(self, tile_op, dst, a, b, p0=0, p1=0, p2=0, p3=0, p4=0, p5=0, p6=0, p7=0,
             dtype=0, adtype=0) -> int:
        self.tasks.append((tile_op | (dtype << 8) | (adtype << 16), dst, a, b, p0, p1, p2, p3,
                           p4, p5, p6, p7))
        return len(self.tasks) - 1

    def ent(self, lane, task, lo=0, hi=0, wait_flag=FLAG_NONE, wait_count=0,
            signal_flag=FLAG_NONE):
        self.lanes[lane].append((task, lo, hi, wait_flag, wait_count, signal_flag, 0, 0))

    def barrier_all(self):
        for lane in range(self.n_lanes):
            self.ent(lane, BARRIER)

    def serialize(self) -> bytes:
        out = bytearray()

        def pad8():
            out.extend(b"\0" * (-len(out) % 8))
        n_entries = sum(len(l) for l in self.lanes)
        out += struct.pack("<IIIIIIIIIIQ", 0x314D5056, 3, len(self.bufs), 0, len(self.consts), 0,
                           len(self.inputs), len(self.outputs), len(self.aux), 0, self.arena)
        for off, size, dt in self.bufs:
            out += struct.pack("<QQII", off, size, dt, 0)
        for ids in (self.inputs, self.outputs):
            for i in ids:
                out += struct.pack("<I", i)
            pad8()
        for dims in (*self.in_dims, *self.out_dims):
            out += struct.pack("<II", len(dims), 0)
            for d in dims:
                out += struct.pack("<Q", d)
        for w in self.aux:
            out += struct.pack("<I", w & 0xFFFFFFFF)
        pad8()
        for bid, data in self.consts:
            out += struct.pack("<II", bid, len(data)) + data
            pad8()
        out += struct.pack("<IIII", len(self.tasks), n_entries, 0, self.n_lanes)
        for t in self.tasks:
            out += struct.pack("<12I", *t)
        off = 0
        for lane, stream in enumerate(self.lanes):
            out += struct.pack("<IIII", off, len(stream), self.root_lens[lane] or len(stream), 0)
            off += len(stream)
        for stream in self.lanes:
            for e in stream:
                out += struct.pack("<8I", *e)
        return bytes(out)
