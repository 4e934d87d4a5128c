"""Token storage -> deterministic causal-LM batches.

Datasets map block indices (or packed span lists) to ``{"input_ids", "targets"}`` of length
``seq_len`` (a window of ``seq_len + 1`` tokens, stride ``seq_len``).  Samplers choose the
epoch order and give every rank an equal, disjoint share of one common deterministic
stream.  Algorithms and defaults follow minitrain/data/dataloader.py:33-669 so that a given
seed yields the same batches; ``DevicePrefetcher`` (pinned staging + copy stream) is an
addition.
"""

from __future__ import annotations

import os
from bisect import bisect_right
from collections import OrderedDict
from collections.abc import Iterator, Sequence
from dataclasses import dataclass
from functools import partial
from pathlib import Path

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, Sampler

from mini_train_sys_b200.data.preprocess import load_manifest
from mini_train_sys_b200.runtime.config import DataConfig


@dataclass(frozen=True)
class PackedBlockSpec:
    """``(global_token_offset, length)`` spans that concatenate to one ``seq_len + 1`` window."""

    segments: tuple[tuple[int, int], ...]


def _as_example(window: torch.Tensor) -> dict[str, torch.Tensor]:
    return {"input_ids": window[:-1], "targets": window[1:]}


def _checked_index(index: int, length: int) -> int:
    if index < 0:
        index += length
    if not 0 <= index < length:
        raise IndexError(index)
    return index


class TokenBlockDataset(Dataset):
    """One in-memory token stream cut into non-overlapping blocks."""

    def __init__(self, tokens: torch.Tensor, seq_len: int) -> None:
        self.tokens = tokens.long()
        self.seq_len = seq_len

    def __len__(self) -> int:
        return max(0, (self.tokens.numel() - 1) // self.seq_len)

    @property
    def sample_ranges(self) -> tuple[tuple[int, int], ...]:
        return ((0, len(self)),) if len(self) else ()

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        begin = _checked_index(idx, len(self)) * self.seq_len
        return _as_example(self.tokens[begin:begin + self.seq_len + 1])


class ShardedTokenBlockDataset(Dataset):
    """Memory-mapped shards addressed as one logical stream; blocks may straddle shard files.

    Only the last incomplete block of the whole split is dropped.  At most ``max_open_shards``
    mappings stay open (LRU, per dataset instance and therefore per loader worker).
    """

    def __init__(self, manifest_path: str | Path, *, split: str, seq_len: int, max_open_shards: int = 8) -> None:
        if seq_len <= 0:
            raise ValueError("seq_len must be positive")
        if max_open_shards <= 0:
            raise ValueError("max_open_shards must be positive")
        self.manifest_path, self.manifest = load_manifest(manifest_path)
        self.root = self.manifest_path.parent
        self.dtype = np.dtype(self.manifest["dtype"])
        info = self.manifest["splits"].get(split)
        if info is None:
            raise ValueError(f"manifest has no split {split!r}")
        self.seq_len = seq_len
        self.max_open_shards = max_open_shards
        self._maps: OrderedDict[int, np.memmap] = OrderedDict()
        files: list[tuple[Path, int]] = []
        stops: list[int] = []
        running = 0
        for rec in info["shards"]:
            path, count = self.root / rec["path"], int(rec["num_tokens"])
            if not path.exists() or path.stat().st_size != count * self.dtype.itemsize:
                raise ValueError(f"token shard size mismatch: {path}")
            if count <= 0:
                continue
            running += count
            files.append((path, count))
            stops.append(running)
        self.total_tokens = running
        self._stops = stops
        self._num_samples = max(0, (running - 1) // seq_len)
        # blocks are grouped by the shard holding their first token (I/O-aware shuffling)
        self.shards: list[tuple[Path, int, int]] = []
        self._sample_ranges: list[tuple[int, int]] = []
        for i, (path, count) in enumerate(files):
            lo_tok = stops[i - 1] if i else 0
            first = min(self._num_samples, -(-lo_tok // seq_len))
            last = min(self._num_samples, -(-stops[i] // seq_len))
            self.shards.append((path, count, max(0, last - first)))
            if first < last:
                self._sample_ranges.append((first, last))

    def __len__(self) -> int:
        return self._num_samples

    @property
    def sample_ranges(self) -> tuple[tuple[int, int], ...]:
        return tuple(self._sample_ranges)

    def __getitem__(self, index: int) -> dict[str, torch.Tensor]:
        begin = _checked_index(index, len(self)) * self.seq_len
        return _as_example(torch.from_numpy(self.read_spans(((begin, self.seq_len + 1),))))

    def read_spans(self, spans: Sequence[tuple[int, int]]) -> np.ndarray:
        out = np.empty(sum(n for _, n in spans), dtype=np.int64)
        cursor = 0
        for start, length in spans:
            done = 0
            while done < length:
                pos = start + done
                shard = bisect_right(self._stops, pos)
                base = self._stops[shard - 1] if shard else 0
                local = pos - base
                take = min(length - done, self.shards[shard][1] - local)
                out[cursor:cursor + take] = self._mapping(shard)[local:local + take]
                cursor += take
                done += take
        return out

    def _mapping(self, shard: int) -> np.memmap:
        hit = self._maps.get(shard)
        if hit is not None:
            self._maps.move_to_end(shard)
            return hit
        path, count, _ = self.shards[shard]
        mapped = np.memmap(path, mode="r", dtype=self.dtype, shape=(count,))
        self._maps[shard] = mapped
        if len(self._maps) > self.max_open_shards:
            _, evicted = self._maps.popitem(last=False)
            handle = getattr(evicted, "_mmap", None)
            if handle is not None:
                handle.close()
        return mapped


class RandomizedDocumentBlockDataset(ShardedTokenBlockDataset):
    """Blocks assembled from an epoch-specific document order; indices are ``PackedBlockSpec``."""

    def __init__(self, manifest_path: str | Path, *, split: str, seq_len: int, max_open_shards: int = 8) -> None:
        super().__init__(manifest_path, split=split, seq_len=seq_len, max_open_shards=max_open_shards)
        meta = self.manifest["splits"][split].get("document_index")
        if meta is None:
            raise ValueError("data.packing='randomized_documents' requires a manifest with a document_index; "
                             "regenerate token shards")
        if meta.get("columns") != ["token_offset", "token_length"]:
            raise ValueError("unsupported document index columns")
        path, entries, dtype = self.root / meta["path"], int(meta["entries"]), np.dtype(meta["dtype"])
        if dtype != np.dtype("<u8") or not path.exists() or path.stat().st_size != entries * 2 * dtype.itemsize:
            raise ValueError(f"document index size or dtype mismatch: {path}")
        table = np.fromfile(path, dtype=dtype).reshape(entries, 2)
        self.document_spans = tuple((int(o), int(n)) for o, n in table)
        expect = 0
        for offset, length in self.document_spans:
            if offset != expect or length <= 0:
                raise ValueError("document index must contain positive contiguous spans")
            expect += length
        if expect != self.total_tokens:
            raise ValueError("document index does not cover the complete token split")

    def __getitem__(self, spec: PackedBlockSpec) -> dict[str, torch.Tensor]:  # type: ignore[override]
        if not isinstance(spec, PackedBlockSpec):
            raise TypeError("randomized document packing requires PackedBlockSpec indices")
        if sum(n for _, n in spec.segments) != self.seq_len + 1:
            raise ValueError("packed block spec must contain exactly seq_len + 1 tokens")
        return _as_example(torch.from_numpy(self.read_spans(spec.segments)))


class _RankShare:
    """Shared rank bookkeeping: equal length for every rank, positions taken modulo world size."""

    def _init_share(self, total: int, rank: int, world_size: int) -> None:
        if not 0 <= rank < world_size:
            raise ValueError(f"rank must be in [0, {world_size}), got {rank}")
        self.rank, self.world_size = rank, world_size
        self.num_samples = total // world_size
        self.total_size = self.num_samples * world_size
        self.epoch = 0

    def __len__(self) -> int:
        return self.num_samples

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def set_start(self, samples: int) -> None:
        """Resume cursor: the next iteration leaves out this rank's first ``samples`` examples of the epoch (they were
        trained on before the interruption); the one after that is a full epoch again."""

        if samples < 0:
            raise ValueError("samples must be non-negative")
        self._start = int(samples)

    def _take_start(self) -> int:
        start, self._start = getattr(self, "_start", 0), 0
        return min(start, self.num_samples)

    def _generator(self) -> torch.Generator:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(self.seed + self.epoch)
        return gen


class ShardAwareBlockSampler(_RankShare, Sampler):
    """Bounded shuffle: shard order, then windows inside a shard, then blocks inside a window."""

    def __init__(self, dataset: Dataset, *, shuffle: bool, seed: int, rank: int = 0, world_size: int = 1,
                 shuffle_window: int = 1024) -> None:
        if shuffle_window <= 0:
            raise ValueError("shuffle_window must be positive")
        ranges = getattr(dataset, "sample_ranges", None)
        if ranges is None:
            ranges = ((0, len(dataset)),) if len(dataset) else ()
        self.sample_ranges = tuple(ranges)
        self._init_share(len(dataset), rank, world_size)
        self.shuffle, self.seed, self.shuffle_window = shuffle, seed, shuffle_window

    def global_order(self) -> Iterator[int]:
        """The stream every rank enumerates identically for the current epoch."""

        if not self.shuffle:
            for lo, hi in self.sample_ranges:
                yield from range(lo, hi)
            return
        gen = self._generator()
        perm = lambda n: torch.randperm(n, generator=gen).tolist()  # noqa: E731
        for r in perm(len(self.sample_ranges)):
            lo, hi = self.sample_ranges[r]
            starts = list(range(lo, hi, self.shuffle_window))
            for w in perm(len(starts)):
                w_lo = starts[w]
                w_hi = min(w_lo + self.shuffle_window, hi)
                for off in perm(w_hi - w_lo):
                    yield w_lo + off

    def __iter__(self) -> Iterator[int]:
        first = self._take_start() * self.world_size      # positions of the common stream that lie before the cursor
        for position, index in enumerate(self.global_order()):
            if position >= self.total_size:
                return
            if position >= first and position % self.world_size == self.rank:
                yield index


class RandomizedDocumentSampler(_RankShare, Sampler):
    """Permute whole documents each epoch, then cut the re-ordered stream into fixed blocks."""

    def __init__(self, dataset: RandomizedDocumentBlockDataset, *, shuffle: bool, seed: int, rank: int = 0,
                 world_size: int = 1) -> None:
        self.dataset = dataset
        self._init_share(len(dataset), rank, world_size)
        self.shuffle, self.seed = shuffle, seed

    def ordered_spans(self) -> list[tuple[int, int]]:
        spans = self.dataset.document_spans
        if not self.shuffle:
            return list(spans)
        order = torch.randperm(len(spans), generator=self._generator()).tolist()
        return [spans[i] for i in order]

    def __iter__(self) -> Iterator[PackedBlockSpec]:
        spans = self.ordered_spans()
        stops = np.cumsum([n for _, n in spans]).tolist()
        seq = self.dataset.seq_len
        for block in range(self.rank + self._take_start() * self.world_size, self.total_size, self.world_size):
            pos = block * seq
            doc = bisect_right(stops, pos)
            inner = pos - (stops[doc - 1] if doc else 0)
            need, pieces = seq + 1, []
            while need:
                offset, length = spans[doc]
                take = min(need, length - inner)
                pieces.append((offset + inner, take))
                need -= take
                doc, inner = doc + 1, 0
            yield PackedBlockSpec(tuple(pieces))


# ---- runtime helpers ---------------------------------------------------------------

def distributed_rank_info() -> tuple[int, int]:
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world < 1:
        raise ValueError(f"WORLD_SIZE must be >= 1, got {world}")
    if not 0 <= rank < world:
        raise ValueError(f"RANK must be in [0, WORLD_SIZE), got rank={rank}, world_size={world}")
    return rank, world


def resolve_data_workers(cfg: DataConfig) -> int:
    """Per-rank worker count: explicit, or an even share of the host budget (one core kept per trainer)."""

    if cfg.num_workers is not None:
        return cfg.num_workers
    ranks_here = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
    me = int(os.environ.get("LOCAL_RANK", "0"))
    spare = max(1, (os.cpu_count() or 1) - ranks_here)
    budget = min(cfg.worker_budget or spare, spare)
    share, extra = divmod(budget, ranks_here)
    return min(cfg.max_workers_per_rank, share + (1 if me < extra else 0))


def _worker_init(worker_id: int, *, local_rank: int, local_world_size: int, workers_per_rank: int,
                 cpu_affinity: bool) -> None:
    torch.set_num_threads(1)
    if not cpu_affinity or not hasattr(os, "sched_getaffinity"):
        return
    cores = sorted(os.sched_getaffinity(0))
    slot = min(local_world_size, len(cores)) + local_rank * workers_per_rank + worker_id
    if slot < len(cores):
        os.sched_setaffinity(0, {cores[slot]})


def load_tokens_from_file(path: str | Path) -> torch.Tensor:
    """Flat token tensor from ``.pt/.pth`` (tensor or {"tokens"|"input_ids"}), ``.npy`` or uint16 ``.bin``."""

    path = Path(path)
    kind = path.suffix.lower()
    if kind in (".pt", ".pth"):
        blob = torch.load(path, map_location="cpu")
        if isinstance(blob, dict):
            blob = blob.get("tokens", blob.get("input_ids"))
        if blob is None:
            raise ValueError(f"{path} did not contain a 'tokens' or 'input_ids' tensor")
        return torch.as_tensor(blob, dtype=torch.long).flatten()
    if kind == ".npy":
        return torch.from_numpy(np.load(path)).long().flatten()
    if kind == ".bin":
        return torch.from_numpy(np.fromfile(path, dtype=np.uint16)).long()
    raise ValueError(f"Unsupported token file format: {path.suffix}")


def _make_loader(dataset: Dataset, cfg: DataConfig, *, batch_size: int, sampler: Sampler) -> DataLoader:
    if len(sampler) == 0:
        raise ValueError(f"Dataset has too few complete blocks for world_size={getattr(sampler, 'world_size', 1)}")
    if cfg.drop_last and len(sampler) < batch_size:
        raise ValueError(f"Dataset provides {len(sampler)} blocks per rank, fewer than batch_size={batch_size} "
                         "with data.drop_last=true")
    workers = resolve_data_workers(cfg)
    ranks_here = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
    options: dict = dict(batch_size=batch_size, sampler=sampler, drop_last=cfg.drop_last, num_workers=workers,
                         pin_memory=cfg.pin_memory and torch.cuda.is_available(),
                         persistent_workers=cfg.persistent_workers and workers > 0)
    if workers > 0:
        options["prefetch_factor"] = cfg.prefetch_factor
        options["worker_init_fn"] = partial(_worker_init, local_rank=int(os.environ.get("LOCAL_RANK", "0")),
                                            local_world_size=ranks_here, workers_per_rank=workers,
                                            cpu_affinity=cfg.worker_cpu_affinity)
    loader = DataLoader(dataset, **options)
    loader.worker_budget = workers * ranks_here
    loader.minitrain_worker_budget = loader.worker_budget
    return loader


def build_dataloader(tokens: torch.Tensor, seq_len: int, batch_size: int, shuffle: bool) -> DataLoader:
    ds = TokenBlockDataset(tokens, seq_len)
    return DataLoader(ds, batch_size=batch_size, sampler=ShardAwareBlockSampler(ds, shuffle=shuffle, seed=0))


def random_token_stream(num_tokens: int, vocab_size: int, seed: int) -> torch.Tensor:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    return torch.randint(low=0, high=vocab_size, size=(num_tokens,), dtype=torch.long, generator=gen)


def build_training_dataloader(cfg: DataConfig, *, seq_len: int, batch_size: int, vocab_size: int, seed: int,
                              split: str = "train") -> DataLoader:
    rank, world = distributed_rank_info()
    if cfg.source == "token_shards":
        randomized = cfg.packing == "randomized_documents"
        cls = RandomizedDocumentBlockDataset if randomized else ShardedTokenBlockDataset
        ds = cls(cfg.path, split=split, seq_len=seq_len, max_open_shards=cfg.max_open_shards)
        if int(ds.manifest["vocab_size"]) > vocab_size:
            raise ValueError(f"dataset vocab_size={ds.manifest['vocab_size']} exceeds model vocab_size={vocab_size}")
        if cfg.tokenizer_fingerprint is not None and cfg.tokenizer_fingerprint != ds.manifest["tokenizer_fingerprint"]:
            raise ValueError("data tokenizer fingerprint does not match configured tokenizer")
        if randomized:
            sampler: Sampler = RandomizedDocumentSampler(ds, shuffle=cfg.shuffle, seed=seed, rank=rank, world_size=world)
        else:
            sampler = ShardAwareBlockSampler(ds, shuffle=cfg.shuffle, seed=seed, rank=rank, world_size=world,
                                             shuffle_window=cfg.shuffle_window)
        return _make_loader(ds, cfg, batch_size=batch_size, sampler=sampler)
    if cfg.source == "random":
        tokens = random_token_stream(cfg.num_tokens, vocab_size, seed)
    elif cfg.source == "tokens":
        tokens = load_tokens_from_file(cfg.path)
    else:
        raise ValueError(f"Unknown data.source: {cfg.source}")
    if tokens.numel() < seq_len + 1:
        raise ValueError(f"Need at least {seq_len + 1} tokens per rank for seq_len={seq_len}, got {tokens.numel()}")
    ds = TokenBlockDataset(tokens, seq_len)
    sampler = ShardAwareBlockSampler(ds, shuffle=cfg.shuffle, seed=seed, rank=rank, world_size=world,
                                     shuffle_window=cfg.shuffle_window)
    return _make_loader(ds, cfg, batch_size=batch_size, sampler=sampler)


class DevicePrefetcher:
    """Wrap a loader: stage the next batch into pinned memory and copy it on a side stream.

    The consumer receives device tensors already in flight; ``record_stream`` ties their
    lifetime to the compute stream.  On CPU devices batches pass through unchanged.
    """

    def __init__(self, loader, device: torch.device) -> None:
        self.loader, self.device = loader, device
        self._stream = torch.cuda.Stream(device) if device.type == "cuda" else None

    def __len__(self) -> int:
        return len(self.loader)

    @property
    def sampler(self):
        return getattr(self.loader, "sampler", None)

    def _stage(self, batch):
        if self._stream is None:
            return batch
        with torch.cuda.stream(self._stream):
            return {k: (v if v.is_pinned() else v.pin_memory()).to(self.device, non_blocking=True)
                    for k, v in batch.items()}

    def __iter__(self):
        it = iter(self.loader)
        try:
            ahead = self._stage(next(it))
        except StopIteration:
            return
        for batch in it:
            ready, ahead = ahead, self._stage(batch)
            yield self._sync(ready)
        yield self._sync(ahead)

    def _sync(self, batch):
        if self._stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._stream)
            for v in batch.values():
                v.record_stream(torch.cuda.current_stream(self.device))
        return batch
