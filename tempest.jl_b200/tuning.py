"""What the library measured while building launches, kept between sessions.

The reference keeps a tuning record per device and toolchain: a tab-separated file of measured seconds by claim, in
`tuning` under `ENV["TEMPEST_CACHE"]` when that is set, appended to as claims are timed and read back when a program
is prepared again, so that a decision reached once is not measured twice (src/Compiler/cover/record.jl:22-32, 60-80).
`TuningRecord` is that for the picks this library makes among its compiled-in variants: which tile form a product
takes (single-CTA tiles of 128 or 256 columns, 256 x 256 tiles by pairs of CTAs), whether its sum is split, how its
results are stored; which of the two forms an attention pullback runs in.  One file per device name; a line is
    family <tab> key <tab> pick <tab> milliseconds
with `pick` as `name=value` pairs joined by `;`.  A later line for the same family and key replaces an earlier one.
"""
import os
import re
import threading


def file_name(name):
    """A device's name as a file name (the reference's rule: anything but letters, digits, `.`, `_`, `-` becomes `_`)."""
    return re.sub(r"[^A-Za-z0-9._-]", "_", name)


def tuning_directory():
    """`tuning` under TEMPEST_CACHE when it is set, else None: nothing is kept unless the caller says where."""
    base = os.environ.get("TEMPEST_CACHE")
    return os.path.join(base, "tuning") if base else None


class TuningRecord:
    def __init__(self, device_name, directory=None):
        directory = directory if directory is not None else tuning_directory()
        self.path = os.path.join(directory, file_name(device_name) + ".b200.tsv") if directory else None
        self.table = {}
        self.written = 0
        self._lock = threading.Lock()
        if self.path and os.path.isfile(self.path):
            with open(self.path) as f:
                for line in f:
                    parts = line.rstrip("\n").split("\t")
                    if len(parts) != 4:
                        continue              # a line cut short by a process that died while writing: skipped
                    family, key, pick, ms = parts
                    try:
                        self.table[(family, key)] = (self._parse(pick), float(ms))
                    except ValueError:
                        continue

    @staticmethod
    def _parse(text):
        pick = {}
        for pair in filter(None, text.split(";")):
            name, value = pair.split("=", 1)
            pick[name] = int(value)
        return pick

    @staticmethod
    def key(*parts):
        return " ".join(str(p) for p in parts)

    def lookup(self, family, key):
        """The pick kept for (family, key), or None."""
        with self._lock:
            kept = self.table.get((family, key))
        return dict(kept[0]) if kept else None

    def keep(self, family, key, pick, milliseconds=0.0):
        """Keeps `pick` (a dict of integers) in memory and appends it to the device's file."""
        pick = {str(k): int(v) for k, v in pick.items()}
        with self._lock:
            self.table[(family, key)] = (pick, float(milliseconds))
            self.written += 1
            if self.path:
                os.makedirs(os.path.dirname(self.path), exist_ok=True)
                text = ";".join(f"{k}={v}" for k, v in sorted(pick.items()))
                with open(self.path, "a") as f:
                    f.write(f"{family}\t{key}\t{text}\t{float(milliseconds)!r}\n")
        return pick
