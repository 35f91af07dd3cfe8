"""Learning from context beyond the window: does the memory carry what a distant part of the document TEACHES (a mapping
applied to new sentences, a function applied to new inputs) or only what it shows verbatim?

Synthetic material in natural held-out sequences.  A teaching block ends with chunk 3 ("beyond": every target chunk lies
past its window) or right before the target chunk ("within": inside the window, the ceiling); "none" has no teaching block.
The test block sits in the target chunk, the same tokens in all three, its scored tokens masked.  Tasks (a fresh draw per
sequence: the weights cannot know the answers):

    span       a 64-token span of another document taught once, read again (cue 16, then every other token scored)
    key1       a passkey, "The special magic number for the lantern is 482913." taught once; test: the cue again, the digits scored
    key4       four such facts with different keys taught together; test: one of them
    lex1_same  a fictional lexicon of 10 nouns -> nonce words in parallel sentences, one sentence per noun; test: the same sentence
    lex1_new   ... test: a new sentence with the same noun
    lex8_same / lex8_new   eight sentences per noun; test: one of them again / a new sentence
    cipher     a letter substitution shown on 40 words; test: 8 new words, the cipher letters scored

Every sequence is written chunk by chunk with the run's own write: the natural pass once, then per task the teaching pass and
the in-window variant; the target chunk is read before it would be written, with the memory on and reset.  Per task and
target, mean CE per scored token:

    recall  = (off - on | beyond) - (off - on | none)        ceiling = (off | beyond) - (off | within)        share = recall / ceiling

``--read l2r``: one read per scored token, everything before it clean and it and everything after it in the chunk masked
(left-to-right decoding with the true prefix); then also, per answer (a run of scored tokens), the exact-match rate under
the memory.  Without a tokenizer (``--synthetic``) the text tasks are replaced by token-level ones of the same structure
(random ids standing for words).  The file holds ``tasks``, ``dist`` (target chunks), ``recall``, ``ceiling``, ``exact``
``[n_seq, n_task, n_target]`` and ``sources``.

    python -m dttt_b200.tools.j_lens.context_learning --ckpt <step dir> --sources name=dir:1.0 --seq_len 32768 --n_per_source 12 \\
        --targets 8,20 [--tasks key1,key4,lex8_new --read l2r] --out cl_32k.npz

Role of the reference's ``tools/j_lens/context_learning.py:1-546``.
"""
from __future__ import annotations

import argparse
import string
import sys
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _cli
from .core import Reader

TASKS = ("span", "key1", "key4", "lex1_same", "lex1_new", "lex8_same", "lex8_new", "cipher")
NOUNS = ("river", "garden", "window", "letter", "bridge", "candle", "forest", "market", "harbor", "village")
FRAMES = ("The {n} was cold.", "She walked to the {n}.", "They painted the {n} last year.", "Nobody remembered the {n}.",
          "A small {n} stood there.", "We could see the {n} from the hill.", "His {n} had been sold.", "The old {n} is gone.",
          "Every {n} looks the same.", "I dreamed of the {n} again.")
OBJECTS = ("lantern", "compass", "violin", "ledger", "anchor", "teapot", "helmet", "basket")
SYLL = ("zor", "vik", "tal", "mur", "esh", "qua", "lin", "dro", "bex", "ony", "pra", "sul")


class Material:
    """A task's teaching tokens, test tokens and the test's scored positions, as ids."""

    def __init__(self, teach: List[int], test: List[int], scored: List[int], answers: List[Tuple[int, int]]):
        self.teach, self.test, self.scored, self.answers = teach, test, scored, answers


class Builder:
    def __init__(self, tokenizer, vocab: int, seed: int):
        self.tok, self.vocab, self.g = tokenizer, vocab, np.random.default_rng(seed)

    def enc(self, text: str) -> List[int]:
        return self.tok(text, add_special_tokens=False)["input_ids"]

    def rand_ids(self, n: int) -> List[int]:
        return self.g.integers(3, self.vocab, size=n).tolist()

    def text_with_answer(self, before: str, answer: str, after: str = "") -> Tuple[List[int], Tuple[int, int]]:
        a, b = self.enc(before), self.enc(answer)
        return a + b + (self.enc(after) if after else []), (len(a), len(a) + len(b))

    def nonce(self) -> str:
        return "".join(self.g.choice(SYLL, size=2, replace=False))

    def build(self, task: str, other_doc: np.ndarray) -> Material:
        if task == "span":
            span = other_doc[:64].tolist()
            sc = list(range(17, 64, 2))
            return Material(span, span, sc, [(i, i + 1) for i in sc])
        if self.tok is None:
            return self.token_level(task)
        if task in ("key1", "key4"):
            n = 1 if task == "key1" else 4
            objs = self.g.choice(OBJECTS, size=n, replace=False)
            nums = [str(int(self.g.integers(100000, 999999))) for _ in range(n)]
            teach = []
            for o, k in zip(objs, nums):
                teach += self.enc(f" The special magic number for the {o} is {k}.")
            test, ans = self.text_with_answer(f" The special magic number for the {objs[0]} is", f" {nums[0]}", ".")
            return Material(teach, test, list(range(*ans)), [ans])
        if task.startswith("lex"):
            reps = 1 if task.startswith("lex1") else 8
            lex = {n: self.nonce() for n in NOUNS}
            teach = []
            for n in NOUNS:
                for f in self.g.choice(len(FRAMES) - 1, size=min(reps, len(FRAMES) - 1), replace=False):
                    teach += self.enc(f" English: {FRAMES[f].format(n=n)} Veltan: {FRAMES[f].format(n=lex[n])}")
                    last_frame = f
            noun = NOUNS[int(self.g.integers(len(NOUNS)))]
            frame = FRAMES[-1] if task.endswith("new") else FRAMES[last_frame]
            if not task.endswith("new"):
                teach += self.enc(f" English: {frame.format(n=noun)} Veltan: {frame.format(n=lex[noun])}")
            pre, post = frame.split("{n}")
            test, ans = self.text_with_answer(f" English: {frame.format(n=noun)} Veltan: {pre}".rstrip(), f" {lex[noun]}", post)
            return Material(teach, test, list(range(*ans)), [ans])
        if task == "cipher":
            letters = list(string.ascii_lowercase)
            perm = dict(zip(letters, self.g.permutation(letters)))
            words = ["horse", "table", "green", "stone", "water", "light", "bread", "chair", "plant", "cloud"] * 4
            teach = []
            for w in words:
                teach += self.enc(f" {w}: " + ", ".join(f"{c} = {perm[c]}" for c in w) + ".")
            test, scored, answers = [], [], []
            for w in ("earth", "night", "bring", "clean", "store", "plate", "grain", "world"):
                for c in w:
                    ids, ans = self.text_with_answer(f" {c} =", f" {perm[c]}", ",")
                    scored += [len(test) + i for i in range(*ans)]
                    answers.append((len(test) + ans[0], len(test) + ans[1]))
                    test += ids
            return Material(teach, test, scored, answers)
        raise ValueError(task)

    def token_level(self, task: str) -> Material:
        """Random ids standing for words: ``cue... answer`` pairs taught once (or eight times) and asked again."""
        n_pairs = {"key1": 1, "key4": 4, "cipher": 12}.get(task, 10)
        reps = 8 if task.startswith("lex8") else 1
        cues = [self.rand_ids(6) for _ in range(n_pairs)]
        answers = [self.rand_ids(2) for _ in range(n_pairs)]
        teach = []
        for _ in range(reps):
            for c, a in zip(cues, answers):
                teach += (self.rand_ids(3) if task.endswith("new") else []) + c + a
        test = cues[0] + answers[0]
        return Material(teach, test, [len(cues[0]), len(cues[0]) + 1], [(len(cues[0]), len(cues[0]) + 2)])


def place(chunk_ids: np.ndarray, block: List[int], at_end: bool) -> Tuple[np.ndarray, int]:
    """Overwrite the end (teaching) or the middle (test) of a chunk with ``block``; returns the chunk and the block's offset."""
    C = len(chunk_ids)
    block = block[-C:] if at_end else block[:C]
    off = C - len(block) if at_end else (C - len(block)) // 2
    out = chunk_ids.copy()
    out[off:off + len(block)] = block
    return out, off


def read_ce(reader: Reader, x: torch.Tensor, scored: np.ndarray, state, mode: str, answers):
    """``(mean CE over the scored tokens, share of the answers exactly right)`` of chunk ``x`` under ``state``."""
    C = reader.C
    m = torch.zeros(1, C, dtype=torch.bool, device=reader.dev)
    m[0, torch.as_tensor(scored)] = True
    shift = 1 if reader.outer_shift else 0
    if mode == "all":
        lg = reader.read(x, m, state)
        ce, sc = reader.slot_ce(lg, x, m)
        top = lg.argmax(-1)
    else:                                                                     # l2r: one read per scored token, the true prefix clean
        ce = torch.zeros(1, C, device=reader.dev)
        top = torch.zeros(1, C, dtype=torch.long, device=reader.dev)
        for s in scored:
            mm = torch.zeros_like(m)
            mm[0, s:] = True
            lg = reader.read(x, mm, state)
            c1, _ = reader.slot_ce(lg, x, m)
            ce[0, s - shift] = c1[0, s - shift]
            top[0, s - shift] = lg[0, s - shift].argmax()
        sc = torch.zeros_like(m)
        sc[0, torch.as_tensor(scored) - shift] = True
    right = [bool(all(int(top[0, i - shift]) == int(x[0, i]) for i in range(a, b))) for a, b in answers]
    return float(ce.sum() / sc.sum().clamp_min(1)), float(np.mean(right)) if right else float("nan")


def measure(reader: Reader, ids: np.ndarray, tasks, targets, read: str, tokenizer, seed: int, log=print) -> dict:
    C, Wn = reader.C, reader.Wn
    n = len(ids)
    rec = np.zeros((n, len(tasks), len(targets)))
    ceil = np.zeros_like(rec)
    exact = np.full_like(rec, np.nan)
    teach_end = 3
    for i in range(n):
        other = ids[(i + 1) % n]
        for ti, task in enumerate(tasks):
            mat = Builder(tokenizer, reader.mc.vocab_size if tokenizer is not None else int(ids.max()) + 1, seed + 1000 * i + ti).build(task, other)
            for tj, tc in enumerate(targets):
                if tc <= teach_end + Wn:
                    raise SystemExit(f"target chunk {tc} is inside the window of the teaching block (chunk {teach_end}, window {Wn})")
                seqs = {}
                for variant in ("beyond", "within", "none"):
                    s = ids[i].copy()
                    tgt, off = place(s[tc * C:(tc + 1) * C], mat.test, at_end=False)
                    s[tc * C:(tc + 1) * C] = tgt
                    if variant != "none":
                        c0 = teach_end if variant == "beyond" else tc - 1
                        blk = mat.teach[-min(teach_end + 1, max(Wn, 1)) * C:]      # fits before chunk 3 and inside a window
                        n_ch = -(-len(blk) // C)
                        for k in range(n_ch):                                # the teaching block ends with chunk c0
                            part = blk[max(0, len(blk) - (k + 1) * C): len(blk) - k * C]
                            s[(c0 - k) * C:(c0 - k + 1) * C], _ = place(s[(c0 - k) * C:(c0 - k + 1) * C], part, at_end=True)
                    seqs[variant] = s
                scored = np.array(mat.scored) + off
                answers = [(a + off, b + off) for a, b in mat.answers]
                vals = {}
                for variant, s in seqs.items():
                    st, _ = reader.write_pass(torch.as_tensor(s[None], device=reader.dev), tc)
                    x = torch.as_tensor(s[None, tc * C:(tc + 1) * C], device=reader.dev)
                    vals[variant, "on"] = read_ce(reader, x, scored, st, read, answers)
                    vals[variant, "off"] = read_ce(reader, x, scored, reader.reset_memory(st), read, answers)
                rec[i, ti, tj] = (vals["beyond", "off"][0] - vals["beyond", "on"][0]) - (vals["none", "off"][0] - vals["none", "on"][0])
                ceil[i, ti, tj] = vals["beyond", "off"][0] - vals["within", "off"][0]
                exact[i, ti, tj] = vals["beyond", "on"][1]
        log(f"[context] sequence {i + 1}/{n}: " + " | ".join(f"{t} {rec[i, k].mean():+.3f}/{ceil[i, k].mean():.3f}" for k, t in enumerate(tasks)))
    return {"recall": rec, "ceiling": ceil, "exact": exact}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.j_lens.context_learning")
    _cli.add_common(ap)
    ap.add_argument("--targets", default="8,20")
    ap.add_argument("--tasks", default=",".join(TASKS))
    ap.add_argument("--read", default="all", choices=("all", "l2r"))
    ap.add_argument("--tokenizer", default="configs/1b_e2e")
    a = ap.parse_args(argv)
    reader, ids, names = _cli.load(a)
    tok = None
    if not a.synthetic:
        from transformers import PreTrainedTokenizerFast
        tok = PreTrainedTokenizerFast.from_pretrained(a.tokenizer)
    tasks = [t for t in a.tasks.split(",") if t]
    targets = [int(x) for x in a.targets.split(",")]
    out = measure(reader, ids, tasks, targets, a.read, tok, a.seed)
    for k, t in enumerate(tasks):
        share = out["recall"][:, k] / np.maximum(out["ceiling"][:, k], 1e-9)
        print(f"[context] {t:10s} share % by target: " + " ".join(f"{tc}: {100 * share[:, j].mean():6.1f}" for j, tc in enumerate(targets))
              + f" | exactly right {100 * np.nanmean(out['exact'][:, k]):.1f}%")
    if a.out:
        np.savez_compressed(a.out, tasks=np.array(tasks), dist=np.array(targets), sources=names, **out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
