"""Benchmark data preparation: prompt formatting, tokenisation and response-only loss masking.

Covers what the reference's scripts/benchmarks/data_processing.py:12-223 does for its benchmark datasets:

* instruct formatting of ``{instruction, input, output}`` records with the Alpaca prompt (with / without an input
  block), the text of the answer appended together with the end-of-sequence token;
* chat-template formatting (a Jinja template rendered per record, ``eos_token`` available to the template);
* tokenisation, with the loss masked (-100) up to and including the response template
  (``"\\n### Response:"`` by default) so that only the answer is learned, which is what TRL's completion-only
  collator does for the reference;
* a cache file per dataset (``cache_<name>.json``) of ``{"input_ids", "labels"}`` rows that
  ``benchmarks/sft_trainer.py --training_data_path`` reads.

No tokenizer can be downloaded here, so any object with ``encode(text) -> List[int]`` and ``eos_token`` works; a
Hugging Face tokenizer loaded from a local directory qualifies, and :class:`ByteTokenizer` is the fallback.

    python -m fms_acceleration_b200.benchmarks.data_processing records.jsonl cache_dir --name alpaca \
        [--tokenizer /path/to/tokenizer] [--chat_template template.jinja] [--max_length 4096]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

IGNORE_INDEX = -100
DEFAULT_RESPONSE_TEMPLATE = "\n### Response:"

PROMPT_WITH_INPUT = (
    "Below is an instruction that describes a task, paired with an input that provides further context. "
    "Write a response that appropriately completes the request.\n\n"
    "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:"
)
PROMPT_NO_INPUT = (
    "Below is an instruction that describes a task. "
    "Write a response that appropriately completes the request.\n\n"
    "### Instruction:\n{instruction}\n\n### Response:"
)


class ByteTokenizer:
    """UTF-8 bytes as tokens (ids 0..255), ``<eos>`` = 256.  Deterministic and dependency-free."""

    eos_token = "<eos>"
    eos_token_id = 256
    vocab_size = 257

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids: List[int] = []
        for i, part in enumerate(text.split(self.eos_token)):
            if i:
                ids.append(self.eos_token_id)
            ids.extend(part.encode("utf-8"))
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        out, buf = [], bytearray()
        for t in ids:
            if t == self.eos_token_id:
                out.append(buf.decode("utf-8", errors="replace") + self.eos_token)
                buf = bytearray()
            else:
                buf.append(t)
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)


def load_tokenizer(path: Optional[str]):
    if not path:
        return ByteTokenizer()
    from transformers import AutoTokenizer  # local directory only: there is no hub access

    return AutoTokenizer.from_pretrained(path, local_files_only=True)


# ------------------------------------------------------------------------------------------- formatting
def format_instruct(record: Dict[str, Any], eos_token: str, input_field: str = "input",
                    output_field: str = "output") -> str:
    prompt = PROMPT_WITH_INPUT if str(record.get(input_field, "") or "") != "" else PROMPT_NO_INPUT
    return prompt.format_map(_Safe(record)) + " " + str(record[output_field]) + eos_token


class _Safe(dict):
    def __missing__(self, key):
        return ""


def format_chat(record: Dict[str, Any], chat_template: str, eos_token: str) -> str:
    """Render ``chat_template`` with ``messages=[record]`` (the convention of the reference's scenario files)."""
    from jinja2 import Environment

    env = Environment(trim_blocks=True, lstrip_blocks=True)
    return env.from_string(chat_template).render(messages=[record], eos_token=eos_token, **record)


def find_subsequence(haystack: Sequence[int], needle: Sequence[int]) -> int:
    """Index of the LAST occurrence of ``needle`` in ``haystack`` or -1."""
    n = len(needle)
    if n == 0:
        return -1
    for i in range(len(haystack) - n, -1, -1):
        if list(haystack[i:i + n]) == list(needle):
            return i
    return -1


def mask_prompt(input_ids: List[int], response_ids: Sequence[int]) -> List[int]:
    """Labels = input ids with everything up to and including the response template set to -100.  A record without
    the template is masked completely (it contributes nothing to the loss), as the completion-only collator does."""
    at = find_subsequence(input_ids, response_ids)
    if at < 0:
        return [IGNORE_INDEX] * len(input_ids)
    cut = at + len(response_ids)
    return [IGNORE_INDEX] * cut + list(input_ids[cut:])


def response_template_ids(tokenizer, response_template: str) -> List[int]:
    """Token ids of the template as they appear INSIDE a text.  Sub-word tokenizers encode a leading newline
    differently at the start of a string, so the template is encoded after a context character and the context's
    ids are cut off."""
    ctx = "a"
    with_ctx = tokenizer.encode(ctx + response_template, add_special_tokens=False)
    only_ctx = tokenizer.encode(ctx, add_special_tokens=False)
    if with_ctx[: len(only_ctx)] == only_ctx:
        return list(with_ctx[len(only_ctx):])
    return list(tokenizer.encode(response_template, add_special_tokens=False))


def build_data_formatting_func(tokenizer=None, formatting: str = "instruct", tokenize: bool = False,
                               input_field: str = "input", dataset_text_field: str = "output",
                               response_template: Optional[str] = DEFAULT_RESPONSE_TEMPLATE,
                               response_field: Optional[str] = None, chat_template: Optional[str] = None,
                               max_length: Optional[int] = None) -> Callable[[Dict[str, Any]], Dict[str, Any]]:
    """Record -> ``{dataset_text_field: text}`` or, with ``tokenize``, ``{"input_ids", "attention_mask", "labels"}``."""
    if tokenize and tokenizer is None:
        raise ValueError("tokenize=True needs a tokenizer")
    eos = getattr(tokenizer, "eos_token", "") or ""
    if tokenize and response_template is None and response_field is None:
        raise ValueError("response_field must be specified if tokenize=True and response_template=None.")
    resp_ids = response_template_ids(tokenizer, response_template) if (tokenize and response_template) else None

    def fmt(record: Dict[str, Any]) -> Dict[str, Any]:
        if chat_template is not None:
            text = format_chat(record, chat_template, eos)
        elif formatting == "instruct":
            text = format_instruct(record, eos, input_field, dataset_text_field)
        else:
            raise ValueError(f"unknown formatting {formatting!r}")
        if not tokenize:
            return {dataset_text_field: text}
        ids = list(tokenizer.encode(text, add_special_tokens=False))
        if resp_ids is not None:
            labels = mask_prompt(ids, resp_ids)
        else:
            # prompt from the template, answer from its own field: mask exactly the prompt
            answer = list(tokenizer.encode(str(record[response_field]), add_special_tokens=False))
            labels = [IGNORE_INDEX] * len(ids) + answer
            ids = ids + answer
        if max_length is not None:
            ids, labels = ids[:max_length], labels[:max_length]
        return {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}

    return fmt


# ------------------------------------------------------------------------------------------- dataset cache
def read_records(path: str) -> List[Dict[str, Any]]:
    with open(path, encoding="utf-8") as fh:
        first = fh.read(1)
        fh.seek(0)
        if first == "[":
            return json.load(fh)
        return [json.loads(line) for line in fh if line.strip()]


def prepare_dataset(records: Iterable[Dict[str, Any]], save_dir: str, name: str, tokenizer=None,
                    chat_template: Optional[str] = None, response_template: Optional[str] = DEFAULT_RESPONSE_TEMPLATE,
                    max_length: Optional[int] = None, overwrite: bool = False) -> str:
    """Format + tokenise ``records`` into ``<save_dir>/cache_<name>.json``; returns the path.  An existing cache is
    kept unless ``overwrite`` (the reference's ``NO_DATA_PROCESSING`` behaviour)."""
    os.makedirs(save_dir, exist_ok=True)
    out = os.path.join(save_dir, f"cache_{name}.json")
    if os.path.exists(out) and not overwrite:
        return out
    tokenizer = tokenizer or ByteTokenizer()
    fmt = build_data_formatting_func(tokenizer, tokenize=True, chat_template=chat_template,
                                     response_template=response_template, max_length=max_length)
    rows = []
    for rec in records:
        row = fmt(rec)
        if any(t != IGNORE_INDEX for t in row["labels"]):
            rows.append({"input_ids": row["input_ids"], "labels": row["labels"]})
    with open(out, "w", encoding="utf-8") as fh:
        json.dump(rows, fh)
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="tokenise an instruct/chat dataset for the benchmarks")
    ap.add_argument("records", help="JSON or JSONL file of records")
    ap.add_argument("save_dir")
    ap.add_argument("--name", default="dataset")
    ap.add_argument("--tokenizer", default=None, help="local tokenizer directory (default: byte tokenizer)")
    ap.add_argument("--chat_template", default=None, help="file holding a Jinja chat template")
    ap.add_argument("--response_template", default=DEFAULT_RESPONSE_TEMPLATE)
    ap.add_argument("--max_length", type=int, default=None)
    ap.add_argument("--overwrite", action="store_true")
    a = ap.parse_args(argv)
    template = open(a.chat_template, encoding="utf-8").read() if a.chat_template else None
    path = prepare_dataset(read_records(a.records), a.save_dir, a.name, load_tokenizer(a.tokenizer), template,
                           a.response_template, a.max_length, a.overwrite)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
