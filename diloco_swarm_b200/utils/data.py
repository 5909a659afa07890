"""Tokenizer, datasets, batching and the microbatch partition.

The reference loads the GPT-2 tokenizer and its datasets from the Hugging Face
hub (src/utils.py:54-57,88-100).  Both are used when reachable; offline the
package falls back to a byte-level tokenizer and to built-in generators:

* ``mikasenghaas/memorize`` / ``memorize``: one sentence repeated 1000 times
  (the reference's memorisation set, tests/test_memorize.py:80);
* ``synthetic:zipf``: token ids iid Zipf(s) over [0, vocab_limit) from a seed.

Local data needs no hub either: ``tokens:<file.npy>`` is a pre-tokenised matrix
of rows of at least seq_length + 1 ids (memory-mapped, so a multi-gigabyte file
costs no memory until its rows are batched), ``text:<file.txt>`` is one example
per non-empty line, tokenised on load.  ``prepare_tokens`` (also the module's
command line) writes such a matrix from a text file, which is what the
reference's data notebook does for its hub datasets (notebooks/1.0-data.ipynb:
pre-tokenised rows of 1025 ids).
"""
from __future__ import annotations

import os
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

MEMORIZE_SENTENCE = "I am a large language model and I can memorize this sentence."


class ByteTokenizer:
    """Byte-level stand-in with the GPT-2 special-token convention (eos = pad = 50256)."""
    eos_token_id = 50256
    pad_token_id = 50256

    def __len__(self) -> int:
        return 50257

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = bytearray()
        for i in (ids.tolist() if hasattr(ids, "tolist") else ids):
            if i < 256:
                out.append(i)
            elif not skip_special_tokens:
                out.extend(b"<|endoftext|>")
        return out.decode("utf-8", errors="replace")


class HFTokenizer:
    def __init__(self, tok):
        self.tok = tok
        self.tok.pad_token = self.tok.eos_token
        self.eos_token_id = tok.eos_token_id
        self.pad_token_id = tok.eos_token_id

    def __len__(self) -> int:
        return len(self.tok)

    def encode(self, text: str) -> List[int]:
        return self.tok(text)["input_ids"]

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self.tok.decode(ids, skip_special_tokens=skip_special_tokens)


def get_tokenizer(prefer_hf: bool = True):
    if prefer_hf and os.environ.get("DSWARM_OFFLINE_TOKENIZER", "0") != "1":
        try:
            os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained("openai-community/gpt2", local_files_only=True)
            return HFTokenizer(tok)
        except Exception:
            pass
    return ByteTokenizer()


def tokenize(text: str, tokenizer, max_length: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Encode one string; with ``max_length`` truncate / right-pad with eos and
    return the matching attention mask (reference: src/utils.py:102-105)."""
    ids = tokenizer.encode(text)
    if max_length is None:
        return {"input_ids": torch.tensor([ids], dtype=torch.long),
                "attention_mask": torch.ones(1, len(ids), dtype=torch.long)}
    ids = ids[:max_length]
    n = len(ids)
    mask = [1] * n + [0] * (max_length - n)
    ids = ids + [tokenizer.pad_token_id] * (max_length - n)
    return {"input_ids": torch.tensor([ids], dtype=torch.long),
            "attention_mask": torch.tensor([mask], dtype=torch.long)}


class TokenDataset:
    """Pre-tokenised sequences of length seq_length + 1 with their masks."""

    def __init__(self, input_ids: torch.Tensor, attention_mask: torch.Tensor):
        assert input_ids.shape == attention_mask.shape
        self.input_ids, self.attention_mask = input_ids, attention_mask

    def __len__(self) -> int:
        return self.input_ids.size(0)

    def rows(self, lo: int, hi: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """ids and mask of rows [lo, hi) as int64 tensors."""
        return self.input_ids[lo:hi], self.attention_mask[lo:hi]

    def select(self, idx) -> "TokenDataset":
        return TokenDataset(self.input_ids[idx], self.attention_mask[idx])

    def train_test_split(self, test_size: float, seed: int, shuffle: bool = True
                         ) -> Tuple["TokenDataset", "TokenDataset"]:
        n = len(self)
        n_test = max(1, int(round(n * test_size))) if test_size > 0 else 0
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(n, generator=g) if shuffle else torch.arange(n)
        return self.select(perm[n_test:]), self.select(perm[:n_test])


class MappedTokenDataset(TokenDataset):
    """Rows of a token matrix on disk.  The matrix (any integer dtype, [N, >= width]) stays
    memory-mapped; ``select`` and the train/validation split only permute an index, and a batch
    copies just its own rows.  ``mask``: optional matrix of the same shape (1 = real token);
    without it every token counts."""

    def __init__(self, ids: np.ndarray, width: int, mask: Optional[np.ndarray] = None,
                 index: Optional[np.ndarray] = None):
        if ids.ndim != 2 or ids.shape[1] < width:
            raise ValueError(f"token matrix of shape {ids.shape} cannot give rows of {width} ids")
        if mask is not None and mask.shape != ids.shape:
            raise ValueError("the mask matrix must have the shape of the token matrix")
        self.ids, self.mask, self.width = ids, mask, width
        self.index = np.arange(ids.shape[0], dtype=np.int64) if index is None else np.asarray(index, dtype=np.int64)

    def __len__(self) -> int:
        return int(self.index.shape[0])

    def rows(self, lo: int, hi: int) -> Tuple[torch.Tensor, torch.Tensor]:
        idx = self.index[lo:hi]
        contiguous = idx.size > 0 and np.all(np.diff(idx) == 1)
        take = (lambda m: m[idx[0]:idx[-1] + 1, :self.width]) if contiguous else (lambda m: m[np.sort(idx), :self.width])
        ids = np.asarray(take(self.ids)).astype(np.int64)
        mask = np.ones_like(ids) if self.mask is None else np.asarray(take(self.mask)).astype(np.int64)
        if not contiguous and idx.size > 0:           # rows were read in file order; put them in index order
            back = np.argsort(np.argsort(idx))
            ids, mask = ids[back], mask[back]
        return torch.from_numpy(ids), torch.from_numpy(mask)

    @property
    def input_ids(self) -> torch.Tensor:          # whole dataset in memory: small sets and tests only
        return self.rows(0, len(self))[0]

    @property
    def attention_mask(self) -> torch.Tensor:
        return self.rows(0, len(self))[1]

    def select(self, idx) -> "MappedTokenDataset":
        idx = idx.numpy() if isinstance(idx, torch.Tensor) else np.asarray(idx, dtype=np.int64)
        return MappedTokenDataset(self.ids, self.width, self.mask, self.index[idx])


def zipf_tokens(num: int, length: int, vocab: int, s: float, seed: int) -> torch.Tensor:
    """iid Zipf(s) ids over [0, vocab): P(k) proportional to (k+1)^-s."""
    w = torch.arange(1, vocab + 1, dtype=torch.float64).pow(-s)
    cdf = torch.cumsum(w / w.sum(), 0)
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(num, length, generator=g, dtype=torch.float64)
    return torch.searchsorted(cdf, u).clamp_(max=vocab - 1).to(torch.long)


def get_dataset(cfg, tokenizer, seed: int, split: str = "train") -> TokenDataset:
    """Build or load the dataset named by ``cfg.path`` as token tensors of
    width ``seq_length + 1`` (inputs and shifted targets share it)."""
    width = cfg.seq_length + 1
    path = cfg.path
    if path.startswith("synthetic:zipf"):
        n = cfg.num_examples or 4096
        ids = zipf_tokens(n, width, cfg.vocab_limit, cfg.zipf_s, seed)
        ds = TokenDataset(ids, torch.ones_like(ids))
    elif path in ("memorize", "mikasenghaas/memorize", "synthetic:memorize"):
        n = cfg.num_examples or 1000
        t = tokenize(MEMORIZE_SENTENCE, tokenizer, max_length=width)
        ds = TokenDataset(t["input_ids"].repeat(n, 1), t["attention_mask"].repeat(n, 1))
    elif path.startswith("tokens:"):
        ds = load_token_file(path[len("tokens:"):], width)
    elif path.startswith("text:"):
        ds = _load_text(path[len("text:"):], tokenizer, width)
    else:
        ds = _load_hf(cfg, tokenizer, width, split)
    if cfg.subset_size < 1.0:
        ds = ds.select(torch.arange(int(len(ds) * cfg.subset_size)))
    return ds


def load_token_file(path: str, width: int) -> MappedTokenDataset:
    """``path``: a .npy matrix of token ids; a sibling ``<stem>.mask.npy`` is used as the mask if present."""
    ids = np.load(path, mmap_mode="r")
    stem = path[:-4] if path.endswith(".npy") else path
    mask = np.load(stem + ".mask.npy", mmap_mode="r") if os.path.exists(stem + ".mask.npy") else None
    return MappedTokenDataset(ids, width, mask)


def _read_examples(path: str) -> List[str]:
    with open(path, encoding="utf-8") as f:
        return [line.strip() for line in f if line.strip()]


def _load_text(path: str, tokenizer, width: int) -> TokenDataset:
    rows = [tokenize(text, tokenizer, width) for text in _read_examples(path)]
    if not rows:
        raise ValueError(f"{path} has no non-empty line")
    return TokenDataset(torch.cat([r["input_ids"] for r in rows]), torch.cat([r["attention_mask"] for r in rows]))


def prepare_tokens(text_path: str, out_path: str, seq_length: int, tokenizer=None, pack: bool = False) -> Tuple[int, int]:
    """Tokenise a text file (one example per non-empty line) into ``out_path`` (.npy, int32 rows of
    seq_length + 1 ids) for ``--data.path tokens:<out_path>``.  Default: one row per line, truncated or
    padded with eos, plus ``<stem>.mask.npy``.  ``pack``: all lines joined by eos and cut into full
    rows (no padding, no mask file; a trailing partial row is dropped).  Returns (rows, width)."""
    tokenizer = tokenizer or get_tokenizer()
    width = seq_length + 1
    stem = out_path[:-4] if out_path.endswith(".npy") else out_path
    examples = _read_examples(text_path)
    if pack:
        stream: List[int] = []
        for text in examples:
            stream.extend(tokenizer.encode(text))
            stream.append(tokenizer.eos_token_id)
        n = len(stream) // width
        ids = np.asarray(stream[:n * width], dtype=np.int32).reshape(n, width)
        if os.path.exists(stem + ".mask.npy"):
            os.remove(stem + ".mask.npy")
    else:
        rows = [tokenize(text, tokenizer, width) for text in examples]
        n = len(rows)
        ids = torch.cat([r["input_ids"] for r in rows]).numpy().astype(np.int32) if rows else np.zeros((0, width), np.int32)
        np.save(stem + ".mask.npy", torch.cat([r["attention_mask"] for r in rows]).numpy().astype(np.uint8)
                if rows else np.zeros((0, width), np.uint8))
    if n == 0:
        raise ValueError(f"{text_path} gives no row of {width} tokens")
    np.save(stem + ".npy", ids)
    return n, width


def _load_hf(cfg, tokenizer, width: int, split: str) -> TokenDataset:
    try:
        from datasets import load_dataset, load_from_disk
    except Exception as e:  # pragma: no cover - depends on the box
        raise RuntimeError(f"dataset {cfg.path!r} needs the `datasets` package: {e}")
    cache = os.path.join(os.environ.get("PERSISTENT_DIR", os.path.expanduser("~/.cache")), "huggingface", cfg.path)
    try:
        dd = load_from_disk(cache)
    except Exception:
        dd = load_dataset(cfg.path)
        os.makedirs(os.path.dirname(cache), exist_ok=True)
        dd.save_to_disk(cache)
    data = dd[split]
    if cfg.tokenize:
        rows = [tokenize(x["text"], tokenizer, width) for x in data]
        ids = torch.cat([r["input_ids"] for r in rows])
        mask = torch.cat([r["attention_mask"] for r in rows])
    else:
        ids = torch.tensor(data["input_ids"], dtype=torch.long)[:, :width]
        mask = torch.tensor(data["attention_mask"], dtype=torch.long)[:, :width]
    return TokenDataset(ids, mask)


def collate(ds: TokenDataset, lo: int, hi: int) -> Dict[str, torch.Tensor]:
    """inputs = ids[:, :-1], targets = ids[:, 1:], mask = mask[:, :-1] (src/utils.py:107-115)."""
    ids, mask = ds.rows(lo, hi)
    return {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(),
            "attention_mask": mask[:, :-1].contiguous()}


class BatchLoader:
    """Sequential, drop-last batches (reference: DataLoader(shuffle=False,
    drop_last=True), src/utils.py:117-118).  With ``pin_memory`` the batch lives
    in page-locked memory so the per-step host-to-device copy is asynchronous."""

    def __init__(self, ds: TokenDataset, batch_size: int, pin_memory: bool = False):
        self.ds, self.batch_size = ds, batch_size
        self.pin = pin_memory and torch.cuda.is_available()

    def __len__(self) -> int:
        return len(self.ds) // self.batch_size

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        for i in range(len(self)):
            b = collate(self.ds, i * self.batch_size, (i + 1) * self.batch_size)
            if self.pin:
                b = {k: v.pin_memory() for k, v in b.items()}
            yield b


def micro_batch_rows(mb: int, micro_batch_size: int) -> slice:
    """Rows of the global batch that form microbatch ``mb``.  Microbatch
    ``k*R0 + i`` is the k-th chunk of first-stage replica i, exactly the
    reference's round-robin chunks ``[k*R0*mbs + i*mbs, +mbs)`` (src/sampler.py:35-38)."""
    return slice(mb * micro_batch_size, (mb + 1) * micro_batch_size)


def get_micro_batches(batch: Dict[str, torch.Tensor], micro_batch_size: int, first_stage_ranks: Sequence[int]
                      ) -> Iterator[Tuple[int, int, Dict[str, torch.Tensor]]]:
    """(root_rank, local_micro_step, micro_batch) for every microbatch of the global batch, in the
    reference's naming (src/utils.py:120-126, src/sampler.py:35-38): first-stage rank i owns the chunks
    k*R0 + i and counts them from 1.  Every rank can evaluate this; only the key would have to travel."""
    n = next(iter(batch.values())).size(0)
    r0 = len(first_stage_ranks)
    for mb in range(n // micro_batch_size):
        rows = micro_batch_rows(mb, micro_batch_size)
        yield first_stage_ranks[mb % r0], mb // r0 + 1, {k: v[rows] for k, v in batch.items()}


class BatchData:
    """A collated batch seen as a dataset of rows (reference: src/sampler.py:6-14)."""

    def __init__(self, batch: Dict[str, torch.Tensor]):
        self.batch = batch

    def __len__(self) -> int:
        return next(iter(self.batch.values())).size(0)

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        return {k: (v[idx] if v is not None else None) for k, v in self.batch.items()}


class BatchSampler:
    """Row indices of a batch that belong to ``rank`` when the rows are dealt out to ``ranks`` in
    round-robin chunks of ``micro_batch_size`` (reference: src/sampler.py:16-39).  The training loop
    itself does not iterate rows: it slices whole microbatches with ``micro_batch_rows``; this class
    states the same partition row by row and is checked against it in the tests."""

    def __init__(self, dataset, rank: int, ranks: Sequence[int], micro_batch_size: int):
        self.n, self.mbs = len(dataset), micro_batch_size
        self.slot, self.width = list(ranks).index(rank), len(ranks)

    def __iter__(self) -> Iterator[int]:
        n_chunks = (self.n + self.mbs - 1) // self.mbs
        for chunk in range(self.slot, n_chunks, self.width):
            yield from range(chunk * self.mbs, min((chunk + 1) * self.mbs, self.n))

    def __len__(self) -> int:
        return sum(1 for _ in self)


def get_dataloader(dataset: TokenDataset, batch_size: int, shuffle: bool = False, pin_memory: bool = False,
                   num_workers: int = 0) -> BatchLoader:
    """The reference's loader factory (src/utils.py:117-118): sequential drop-last batches.  Batches are
    slices of one resident tensor, so there are no worker processes to start (``num_workers`` is accepted
    and ignored); ``shuffle`` permutes the dataset once, seeded, before batching."""
    if shuffle:
        g = torch.Generator().manual_seed(0)
        dataset = dataset.select(torch.randperm(len(dataset), generator=g).tolist())
    return BatchLoader(dataset, batch_size, pin_memory=pin_memory)


def get_num_steps(max_steps: int, max_epochs: int, num_examples: int, batch_size: int) -> int:
    """Whichever of max_steps / max_epochs is reached first (src/utils.py:145-152)."""
    if num_examples < batch_size:
        raise ValueError("Number of examples must be at least batch size")
    if not (max_steps > 0 or max_epochs > 0):
        raise ValueError("Specify at least one of `max_steps` and `max_epochs`")
    per_epochs = num_examples // batch_size * max_epochs
    if max_epochs == -1:
        return max_steps
    if max_steps == -1:
        return per_epochs
    return min(max_steps, per_epochs)


def get_train_setup(steps: int, batch_size: int, seq_length: int, micro_batch_size: int, num_examples: int):
    tokens_per_step = batch_size * seq_length
    return {"steps": steps, "batch_size": batch_size, "seq_length": seq_length,
            "micro_batch_size": micro_batch_size, "tokens_per_step": tokens_per_step,
            "total_tokens": steps * tokens_per_step,
            "avg_token_repetitions": steps * tokens_per_step / max(1, num_examples * seq_length),
            "grad_accumulation_steps": batch_size // micro_batch_size if micro_batch_size > 0 else 1}


def _main() -> None:
    import argparse
    ap = argparse.ArgumentParser(description="Tokenise a text file into a token matrix for --data.path tokens:<file>")
    ap.add_argument("--text", required=True, help="text file, one example per non-empty line")
    ap.add_argument("--out", required=True, help="output .npy file")
    ap.add_argument("--seq-length", type=int, default=1024)
    ap.add_argument("--pack", action="store_true", help="join the lines with eos and cut full rows instead of padding")
    a = ap.parse_args()
    n, width = prepare_tokens(a.text, a.out, a.seq_length, pack=a.pack)
    print(f"wrote {n} rows of {width} token ids to {a.out}")


if __name__ == "__main__":
    _main()
