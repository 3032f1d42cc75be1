"""Slot data generators (python/paddle/distributed/fleet/data_generator/data_generator.py): turn raw text lines into
the ``<count> <v1> <v2> ...`` per-slot format that the slot datasets read."""
from __future__ import annotations

import sys


class DataGenerator:
    def __init__(self):
        self._proto_info = None
        self.batch_size_ = 32

    def set_batch(self, batch_size):
        self.batch_size_ = batch_size

    def generate_sample(self, line):
        raise NotImplementedError("Please rewrite this function to return a generator of [(name, [values]), ...]")

    def generate_batch(self, samples):
        def local_iter():
            yield from samples
        return local_iter

    def _gen_str(self, line):
        raise NotImplementedError

    def _run(self, lines, out):
        batch = []
        for line in lines:
            for sample in self.generate_sample(line)():
                if sample is None:
                    continue
                batch.append(sample)
                if len(batch) == self.batch_size_:
                    for s in self.generate_batch(batch)():
                        out.write(self._gen_str(s))
                    batch = []
        if batch:
            for s in self.generate_batch(batch)():
                out.write(self._gen_str(s))

    def run_from_stdin(self):
        self._run(sys.stdin, sys.stdout)

    def run_from_memory(self):
        self._run([None], sys.stdout)


def _check(line):
    if isinstance(line, zip):
        line = list(line)
    if not isinstance(line, (list, tuple)):
        raise ValueError("the output of process() must be in list or tuple type"
                         "Example: [('words', [1926, 08, 17]), ('label', [1])]")
    return line


class MultiSlotDataGenerator(DataGenerator):
    def _gen_str(self, line):
        line = _check(line)
        first = self._proto_info is None
        if first:
            self._proto_info = []
        elif len(line) != len(self._proto_info):
            raise ValueError("the complete field set of two given line are inconsistent.")
        parts = []
        for i, (name, elements) in enumerate(line):
            if not isinstance(name, str):
                raise ValueError(f"name {type(name)} must be in str type")
            if not isinstance(elements, list):
                raise ValueError(f"elements {type(elements)} must be in list type")
            if not elements:
                raise ValueError("the elements of each field can not be empty, you need padding it in process().")
            kind = "float" if any(isinstance(e, float) for e in elements) else "uint64"
            if first:
                self._proto_info.append((name, kind))
            else:
                if name != self._proto_info[i][0]:
                    raise ValueError(f"the field name of two given line are not match: require<{self._proto_info[i][0]}>, get<{name}>.")
                if kind == "float" and self._proto_info[i][1] == "uint64":
                    self._proto_info[i] = (name, "float")
            parts.append(" ".join([str(len(elements))] + [str(e) for e in elements]))
        return " ".join(parts) + "\n"


class MultiSlotStringDataGenerator(DataGenerator):
    def _gen_str(self, line):
        line = _check(line)
        parts = []
        for name, elements in line:
            parts.append(" ".join([str(len(elements))] + list(elements)))
        return " ".join(parts) + "\n"
