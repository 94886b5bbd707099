"""Expert banks on disk -> pinned host banks: reader, writer and loaders of the reference's repacked weight directory.

The directory format is the one ``freetoken/python/freetoken/checkpoint/ftw.py:1-31,123-176`` defines (index
``freetoken_weight.json`` + shard files ``freetoken-NNNNN.ftw``): all tensors form one logical byte region; every
tensor starts on a 4096-byte boundary and is padded to the next one; the region is cut into shard files of at most
``shard_limit`` bytes at 4096-byte boundaries; a tensor that fits a shard is never split.  Expert banks are entries
of kind ``experts_bank`` named like the reference's schema (``moe/offload_cache.py:87-94``: ``gate_up_packed,
gate_up_scale, gate_up_global, down_packed, down_scale, down_global`` for NVFP4), either one flat
``[layers * experts, ...]`` region per bank or one ``name#Llllll`` entry per (bank, layer)
(``checkpoint/ftw.py:498-531``).  Files written here are readable by the reference and the other way round (the
tests hold a directory written by the reference's own writer).

Two loaders sit on the reader:

  * :func:`load_banks` -- the reference's contract (``load_ftw_banks``, ``checkpoint/ftw.py:487-728``): per role one
    ``[experts, ...]`` host bank per layer, filled, then pinned;
  * :func:`load_records` -- the layout this package's slot cache prefers: per layer ONE bank ``[experts,
    record_bytes]`` with an expert's six pieces back to back, so that a cache miss is one contiguous copy.  The file
    bytes are read straight into the strided role views of the record bank; nothing is staged twice.
"""
from __future__ import annotations

import bisect
import json
import math
import mmap
import os
import re
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import torch

from .host_banks import HostBank

INDEX_NAME = "freetoken_weight.json"
FORMAT_TAG, FORMAT_VERSION = "freetoken_weight", 1
ALIGN = 4096
DEFAULT_SHARD_LIMIT = 8 << 30
BANK_KIND = "experts_bank"
NUM_LAYERS_KEY = "expert_bank_num_layers"
# role used by the kernels <-> bank name stored in the files (``moe/legacy_format.py:7-14``)
STORED_NAME = {"gate_up": "gate_up_packed", "gate_up_scale": "gate_up_scale", "gate_up_global": "gate_up_global",
               "down": "down_packed", "down_scale": "down_scale", "down_global": "down_global"}
ROLE_OF = {"gate_up_packed": "gate_up", "gate_up_blocks": "gate_up", "gate_up_scales": "gate_up_scale",
           "down_packed": "down", "down_blocks": "down", "down_scales": "down_scale"}
_LAYER_NAME = re.compile(r"^(?P<base>.+)#L(?P<layer>\d{5})$")


class BankIndexError(ValueError):
    """The index does not describe a byte layout this reader can interpret exactly."""


def shard_file_name(i: int) -> str:
    return "freetoken-%05d.ftw" % i


def layer_entry_name(bank_name: str, layer: int) -> str:
    return "%s#L%05d" % (bank_name, layer)


def _round_up(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def _elsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _nat(v) -> bool:
    return type(v) is int and v >= 0


def read_index(path: str) -> dict:
    """Load and validate the index; every number the reader later trusts is checked against the others."""
    file = os.path.join(path, INDEX_NAME)

    def need(ok: bool, what: str) -> None:
        if not ok:
            raise BankIndexError(f"{file}: {what}")

    with open(file) as f:
        idx = json.load(f)
    need(type(idx) is dict, "the index is not an object")
    need(idx.get("format") == FORMAT_TAG, "wrong format tag")
    need(type(idx.get("version")) is int and idx["version"] == FORMAT_VERSION, f"unsupported version {idx.get('version')!r}")
    need(type(idx.get("align")) is int and idx["align"] == ALIGN, f"align must be {ALIGN}")
    limit, total = idx.get("shard_limit"), idx.get("total_bytes")
    need(_nat(limit) and limit > 0 and limit % ALIGN == 0, "bad shard_limit")
    need(_nat(total) and total % ALIGN == 0, "bad total_bytes")
    need(type(idx.get("shards")) is list and type(idx.get("tensors")) is list, "shards and tensors must be lists")
    pos = 0
    for i, sh in enumerate(idx["shards"]):
        need(type(sh) is dict and sh.get("file") == shard_file_name(i), f"shard {i}: unexpected file name")
        need(_nat(sh.get("global_off")) and sh["global_off"] == pos, f"shard {i}: gap or overlap")
        need(_nat(sh.get("nbytes")) and sh["nbytes"] % ALIGN == 0 and sh["nbytes"] <= limit, f"shard {i}: bad size")
        pos += sh["nbytes"]
    need(pos == total, f"shards cover {pos} bytes of {total}")
    seen, floor = set(), 0
    for t in idx["tensors"]:
        need(type(t) is dict and type(t.get("name")) is str and t["name"] != "", "tensor without a name")
        name = t["name"]
        need(name not in seen, f"duplicate tensor {name!r}")
        seen.add(name)
        need(type(t.get("kind")) is str and t["kind"] != "", f"{name}: no kind")
        dtype = getattr(torch, t["dtype"], None) if type(t.get("dtype")) is str else None
        need(isinstance(dtype, torch.dtype), f"{name}: unknown dtype {t.get('dtype')!r}")
        shape, off, n = t.get("shape"), t.get("global_off"), t.get("nbytes")
        need(type(shape) is list and all(_nat(d) for d in shape), f"{name}: bad shape")
        need(_nat(n) and n == math.prod(shape) * _elsize(dtype), f"{name}: nbytes does not match dtype x shape")
        need(_nat(off) and off % ALIGN == 0, f"{name}: unaligned offset")
        need(off >= floor, f"{name}: overlaps the tensor before it")
        need(off + n <= total, f"{name}: reaches past the region")
        floor = _round_up(off + n)
    return idx


def is_bank_directory(path: str) -> bool:
    return os.path.isfile(os.path.join(path, INDEX_NAME))


class BankFileWriter:
    """Appends tensors to the byte region, opening a new shard whenever the current one is full (or a tensor that
    fits a whole shard would straddle the boundary).  ``finalize(meta)`` writes the index atomically."""

    def __init__(self, out_dir: str, shard_limit: int = DEFAULT_SHARD_LIMIT):
        if shard_limit <= 0 or shard_limit % ALIGN:
            raise ValueError("shard_limit must be a positive multiple of %d" % ALIGN)
        os.makedirs(out_dir, exist_ok=True)
        self.out_dir, self.limit = out_dir, shard_limit
        self.tensors: list[dict] = []
        self.shards: list[dict] = []
        self.pos = 0            # region offset of the next byte
        self._file = None
        self._used = 0          # bytes in the open shard

    def _close_shard(self) -> None:
        if self._file is not None:
            self.shards.append({"file": shard_file_name(len(self.shards)), "global_off": self.pos - self._used,
                                "nbytes": self._used})
            self._file.close()
            self._file = None

    def _open_shard(self) -> None:
        self._close_shard()
        self._file = open(os.path.join(self.out_dir, shard_file_name(len(self.shards))), "wb")
        self._used = 0

    def _append(self, data: memoryview) -> None:
        done = 0
        while done < len(data):
            if self._file is None or self._used == self.limit:
                self._open_shard()
            n = min(len(data) - done, self.limit - self._used)
            self._file.write(data[done:done + n])
            done, self._used, self.pos = done + n, self._used + n, self.pos + n

    def add_tensor(self, name: str, tensor: torch.Tensor, kind: str = "weight") -> None:
        t = tensor.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8)
        n = raw.numel()
        if self._file is None or (n <= self.limit and self._used + n > self.limit):
            self._open_shard()
        self.tensors.append({"name": name, "kind": kind, "dtype": str(t.dtype).removeprefix("torch."),
                             "shape": list(t.shape), "global_off": self.pos, "nbytes": n})
        self._append(memoryview(raw.numpy()))
        pad = _round_up(self.pos) - self.pos
        if pad:
            self._append(memoryview(bytes(pad)))

    def finalize(self, meta: dict | None = None) -> dict:
        self._close_shard()
        index = {"format": FORMAT_TAG, "version": FORMAT_VERSION, "align": ALIGN, "shard_limit": self.limit,
                 "total_bytes": self.pos, "tensors": self.tensors, "shards": self.shards, **(meta or {})}
        tmp = os.path.join(self.out_dir, INDEX_NAME + ".tmp")
        with open(tmp, "w") as f:
            json.dump(index, f)
        os.replace(tmp, os.path.join(self.out_dir, INDEX_NAME))
        return index


class BankFileReader:
    """Random access to the byte region.  A request [offset, offset + nbytes) is split at shard boundaries (binary
    search over the shard offsets) and every piece is read with positional reads straight into the destination
    buffer, large pieces by several threads.  With ``direct=True`` the shards are opened with O_DIRECT when the file
    system takes it (destination, offset and length must then be 4096-aligned: ``read_window`` does the rounding);
    otherwise the page cache is used."""

    CHUNK = 8 << 20

    def __init__(self, path: str, direct: bool = False, workers: int = 8):
        self.dir = path
        self.index = read_index(path)
        self.shards = self.index["shards"]
        self.tensors = {t["name"]: t for t in self.index["tensors"]}
        self._starts = [s["global_off"] for s in self.shards]
        self._fds: dict[int, int] = {}
        self._flags = os.O_RDONLY
        self.direct = False
        if direct and hasattr(os, "O_DIRECT") and self.shards:
            try:
                os.close(os.open(os.path.join(path, self.shards[0]["file"]), os.O_RDONLY | os.O_DIRECT))
                self._flags |= os.O_DIRECT
                self.direct = True
            except OSError:
                pass
        self.workers = workers

    def meta(self, key: str, default=None):
        return self.index.get(key, default)

    def entries(self, *kinds: str) -> list[dict]:
        return [t for t in self.index["tensors"] if not kinds or t["kind"] in kinds]

    def close(self) -> None:
        for fd in self._fds.values():
            os.close(fd)
        self._fds.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _fd(self, shard: int) -> int:
        if shard not in self._fds:
            self._fds[shard] = os.open(os.path.join(self.dir, self.shards[shard]["file"]), self._flags)
        return self._fds[shard]

    def pieces(self, offset: int, nbytes: int):
        """(shard, offset in the shard file, offset in the destination, length) covering the request."""
        if offset < 0 or nbytes < 0 or offset + nbytes > self.index["total_bytes"]:
            raise ValueError("range outside the region")
        out, done = [], 0
        i = max(0, bisect.bisect_right(self._starts, offset) - 1)
        while done < nbytes:
            sh = self.shards[i]
            inside = offset + done - sh["global_off"]
            n = min(nbytes - done, sh["nbytes"] - inside)
            out.append((i, inside, done, n))
            done += n
            i += 1
        return out

    def read_range(self, dest: memoryview, offset: int, nbytes: int) -> None:
        """Fill ``dest[:nbytes]`` with region bytes [offset, offset + nbytes)."""
        jobs = []
        for shard, inside, at, n in self.pieces(offset, nbytes):
            self._fd(shard)  # opened here, on one thread
            for c in range(0, n, self.CHUNK):
                jobs.append((shard, inside + c, at + c, min(self.CHUNK, n - c)))

        def run(job):
            shard, inside, at, n = job
            fd, got = self._fds[shard], 0
            while got < n:
                r = os.preadv(fd, [dest[at + got:at + n]], inside + got)
                if r <= 0:
                    raise OSError(f"{self.shards[shard]['file']}: file ends at {inside + got}, {n - got} bytes short")
                got += r

        if len(jobs) <= 1:
            for j in jobs:
                run(j)
        else:
            with ThreadPoolExecutor(self.workers) as pool:
                list(pool.map(run, jobs))

    def read_window(self, offset: int, nbytes: int) -> tuple[mmap.mmap, int]:
        """The 4096-aligned window enclosing [offset, offset + nbytes) in a fresh page-aligned buffer (legal for
        O_DIRECT: the region is padded to 4096, so the window never leaves it); returns (buffer, offset of the
        requested bytes inside it)."""
        lo = offset // ALIGN * ALIGN
        hi = _round_up(offset + nbytes)
        buf = mmap.mmap(-1, max(hi - lo, ALIGN))
        self.read_range(memoryview(buf), lo, hi - lo)
        return buf, offset - lo

    def tensor(self, name: str) -> torch.Tensor:
        """One entry as a host tensor (its own memory)."""
        e = self.tensors[name]
        dtype = getattr(torch, e["dtype"])
        buf, head = self.read_window(e["global_off"], e["nbytes"])
        t = torch.frombuffer(buf, dtype=torch.uint8, count=e["nbytes"], offset=head).clone() if e["nbytes"] else \
            torch.empty(0, dtype=torch.uint8)
        return t.view(dtype).view(*e["shape"]) if e["shape"] else t.view(dtype).view(())


# ---------------------------------------------------------------------------------------------------------------
def write_expert_banks(out_dir: str, layers: list[dict[str, torch.Tensor]], quant_format: str = "nvfp4",
                       per_layer: bool = True, shard_limit: int = DEFAULT_SHARD_LIMIT, extra: dict | None = None) -> dict:
    """Write per-layer role tensors (``[experts, ...]`` each) as ``experts_bank`` entries under the stored names:
    one entry per (bank, layer) (``per_layer``) or one flat ``[layers * experts, ...]`` region per bank."""
    w = BankFileWriter(out_dir, shard_limit)
    for role in layers[0]:
        stored = STORED_NAME.get(role, role)
        if per_layer:
            for l, banks in enumerate(layers):
                w.add_tensor(layer_entry_name(stored, l), banks[role], BANK_KIND)
        else:
            w.add_tensor(stored, torch.cat([b[role] for b in layers], dim=0), BANK_KIND)
    return w.finalize({"quant_format": quant_format, NUM_LAYERS_KEY: len(layers), **(extra or {})})


@dataclass
class LoadedBanks:
    quant_format: str | None
    sources: dict[str, list[torch.Tensor]]   # role -> per layer [experts, ...] (views of ``host_banks``)
    host_banks: list[HostBank]
    num_layers: int
    num_experts: int


def _bank_plan(reader: BankFileReader, num_layers: int) -> dict[str, list[tuple[int, int, tuple[int, ...], torch.dtype]]]:
    """role -> per layer (region offset, nbytes, [experts, ...] shape, dtype), from either on-disk row layout."""
    meta_layers = reader.meta(NUM_LAYERS_KEY)
    if meta_layers is not None and meta_layers != num_layers:
        raise RuntimeError(f"the directory was written for {meta_layers} MoE layers, the caller expects {num_layers}")
    flat, split = {}, {}
    for e in reader.entries(BANK_KIND):
        m = _LAYER_NAME.match(e["name"])
        if m is None:
            flat[e["name"]] = e
        else:
            split.setdefault(m.group("base"), {})[int(m.group("layer"))] = e
    both = set(flat) & set(split)
    if both:
        raise BankIndexError(f"banks stored both flat and per layer: {sorted(both)}")
    plan = {}
    for name, e in flat.items():
        rows, *rest = e["shape"]
        if rows % num_layers:
            raise BankIndexError(f"{name}: {rows} rows do not divide into {num_layers} layers")
        per = e["nbytes"] // num_layers
        dtype = getattr(torch, e["dtype"])
        plan[ROLE_OF.get(name, name)] = [(e["global_off"] + l * per, per, (rows // num_layers, *rest), dtype)
                                         for l in range(num_layers)]
    for name, by_layer in split.items():
        if sorted(by_layer) != list(range(num_layers)):
            raise BankIndexError(f"{name}: layers {sorted(by_layer)} on disk, expected 0..{num_layers - 1}")
        plan[ROLE_OF.get(name, name)] = [(by_layer[l]["global_off"], by_layer[l]["nbytes"], tuple(by_layer[l]["shape"]),
                                          getattr(torch, by_layer[l]["dtype"])) for l in range(num_layers)]
    return plan


def load_banks(path: str, num_layers: int, pin: bool = True, direct: bool = False, workers: int = 8) -> LoadedBanks | None:
    """Per role and layer one host bank ``[experts, ...]`` (lazy huge-page buffer -> filled from the files -> pinned).
    ``None`` when the directory holds no expert banks."""
    with BankFileReader(path, direct=direct, workers=workers) as reader:
        plan = _bank_plan(reader, num_layers)
        if not plan:
            return None
        sources, keep = {}, []
        for role, per_layer in plan.items():
            sources[role] = []
            for off, nbytes, shape, dtype in per_layer:
                lo = off // ALIGN * ALIGN                      # a layer of a flat region may start inside a block
                bank = HostBank((_round_up(off + nbytes) - lo,), torch.uint8)
                reader.read_range(memoryview(bank._buf), lo, _round_up(off + nbytes) - lo)
                sources[role].append(bank.tensor[off - lo:off - lo + nbytes].view(dtype).view(*shape))
                keep.append(bank)
        quant = reader.meta("quant_format")
    if pin:
        for b in keep:
            b.pin()
    experts = next(iter(sources.values()))[0].shape[0]
    return LoadedBanks(quant, sources, keep, num_layers, experts)


def load_records(path: str, num_layers: int, layout: dict, pin: bool = True, workers: int = 8) -> tuple[list[torch.Tensor], list[HostBank]]:
    """Per layer one host bank ``[experts, record_bytes]`` in the slot cache's record layout (the six pieces of an
    expert back to back, in the order of ``layout``), filled straight from the files and pinned.  Returns the
    tensors for ``SlotCache.set_record_sources`` and the banks that own their memory."""
    from .slot_cache import SlotCache

    rb = SlotCache.record_bytes(layout)
    with BankFileReader(path, workers=workers) as reader:
        plan = _bank_plan(reader, num_layers)
        missing = [r for r in layout if r not in plan]
        if missing:
            raise BankIndexError(f"the directory lacks the banks {missing}")
        experts = plan[next(iter(layout))][0][2][0]
        records, keep = [], []
        for l in range(num_layers):
            bank = HostBank((experts, rb), torch.uint8)
            views = SlotCache.record_views(bank.tensor, layout)
            for role, spec in layout.items():
                off, nbytes, shape, dtype = plan[role][l]
                if shape != (experts, *spec.shape) or dtype != spec.dtype:
                    raise BankIndexError(f"{role} of layer {l}: {shape} {dtype} on disk, the kernel wants "
                                         f"{(experts, *spec.shape)} {spec.dtype}")
                buf, head = reader.read_window(off, nbytes)
                views[role].copy_(torch.frombuffer(buf, dtype=torch.uint8, count=nbytes, offset=head).view(dtype).view(*shape))
            records.append(bank.tensor)
            keep.append(bank)
    if pin:
        for b in keep:
            b.pin()
    return records, keep


__all__ = ["BankFileWriter", "BankFileReader", "BankIndexError", "read_index", "is_bank_directory", "write_expert_banks",
           "load_banks", "load_records", "LoadedBanks", "layer_entry_name", "shard_file_name", "INDEX_NAME", "ALIGN",
           "STORED_NAME", "ROLE_OF", "BANK_KIND"]
