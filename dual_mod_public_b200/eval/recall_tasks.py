"""Document-grounded recall tasks and needle-in-a-haystack tasks, as plain protocol code.

Two task families the evaluation of the reference adds to the stock harness:

  recall     six reading-comprehension / extraction sets (SWDE, FDA, SQuAD, TriviaQA, NQ, DROP) under
             the "read the document, then answer" protocol at a 2k-token input: the document is cut to a
             window of `context_length - answer_length` tokens CENTRED on the first occurrence of the
             answer (sets without an answer key keep the document head), the prompt is
             "<document>. <question>" (extraction sets: "<document>. <Key>:"), generation is greedy up to
             48 tokens or a newline, and the score is a case-insensitive "contains"
  needles    jsonl files written by the official RULER generators (one folder per task and length);
             prompt = input + answer prefix, 128 new tokens, score = share of reference strings found

Everything here works on plain dicts and any object with `generate_until` (the adapters of
`lm_eval_adapter.py`), so a folder of jsonl files is enough to run a task:

    docs = load_jsonl("fda.jsonl")
    print(run_recall(lm, "fda", docs, tokenizer=lm.tok))

`harness_tasks()` additionally wraps the recall tasks as `lm_eval` task classes when that package is
installed (they then load their datasets from the hub by the names in `RECALL`).

Reference parity: lm/eval/based_tasks/jrt_tasks.py:44-234 (window cut, prompts, metric, shard selection),
lm/eval/based_tasks/ruler_official.py:1-33 and the ruler_off_niah_*.yaml files (needle tasks).
"""

from __future__ import annotations

import json
import os
import re

# name: (hub dataset, key of the document text, keys whose first match centres the window, prompt kind)
RECALL = {
    "squad": ("hazyresearch/based-squad", "text", ("value",), "completion"),
    "fda": ("hazyresearch/based-fda", "text", ("key", "value"), "extract"),
    "swde": ("hazyresearch/based-swde-v2", "text", ("key", "value"), "extract"),
    "triviaqa": ("hazyresearch/based_triviaqa", "context", (), "qa"),
    "nq": ("hazyresearch/based_nq_2048", "context", ("answers",), "qa"),
    "drop": ("hazyresearch/based_drop", "context", (), "qa"),
}
NEEDLE_TASKS = ("niah_single_1", "niah_single_2", "niah_single_3",
                "niah_multikey_1", "niah_multikey_2", "niah_multikey_3")
GEN_RECALL = {"until": ["\n"], "max_gen_toks": 48}
GEN_NEEDLE = {"until": [], "max_gen_toks": 128}
SUMMARY_MARK = "Summary of information above..."


def load_jsonl(path):
    return [json.loads(line) for line in open(path) if line.strip()]


def shard(docs, spec=None):
    """`i/n` keeps documents i, i+n, i+2n, ... (default: the JRT_SHARD environment variable)."""
    spec = spec if spec is not None else os.environ.get("JRT_SHARD", "")
    if not spec:
        return list(docs)
    i, n = (int(v) for v in spec.split("/"))
    return [d for j, d in enumerate(docs) if j % n == i]


def contains_score(prediction, labels):
    return max(int(re.search(re.escape(l), prediction, re.IGNORECASE) is not None) for l in labels)


def _first_match(text, needle):
    m = re.search(re.escape(needle), text, re.IGNORECASE)
    return m.start() if m else -1


def _ids(tok, text):
    out = tok(text, add_special_tokens=True)["input_ids"] if callable(tok) else tok.encode(text)
    return list(out)


def cut_to_answer(doc, text_key, answer_keys, tok, context_length=2048, answer_length=50, keep_lead=False):
    """Copy of `doc` whose text is the token window of `context_length - answer_length` tokens around
    the answer (half before it, the rest after).  No answer keys: the window starts at the head.  An
    answer that is empty or a single character returns None (the protocol drops such documents from
    the cut and uses them whole)."""
    budget = context_length - answer_length
    text = doc[text_key] if keep_lead else doc[text_key].strip()
    ids = _ids(tok, text)
    at = -1
    for key in answer_keys:
        ans = doc[key][0] if isinstance(doc[key], list) else doc[key]
        if len(ans) <= 1:
            return None
        p = _first_match(text, ans)
        if p >= 0 and (at < 0 or p < at):
            at = p
    if at < 0:
        for ans in doc.get("alt_answers", ()):
            at = _first_match(text, ans)
            if at >= 0:
                break
    if not answer_keys:
        at = 0
    centre = len(_ids(tok, text[:at])) if at >= 0 else len(_ids(tok, text[:-1]))
    if at < 0 and "tok_pos" in doc and centre > budget:
        centre = int(doc["tok_pos"])
    start = max(0, centre - budget // 2)
    end = min(len(ids), centre + budget - (centre - start))
    out = dict(doc)
    out[text_key] = tok.decode(ids[start:end], skip_special_tokens=True)
    return out


def _strip_question(text, question):
    while question and text.lower().endswith(question.lower()):
        text = text[:-len(question)]
    return text


def env_options():
    """Protocol switches from the environment: JRT_CONTEXT_LENGTH / JRT_ANSWER_LENGTH (window size), JRT_NO_STRIP=1
    (keep the document's leading whitespace), JRT_PREPEND_SPACES=N (strip, then prepend N spaces)."""
    e = os.environ
    return dict(context_length=int(e.get("JRT_CONTEXT_LENGTH", 2048)), answer_length=int(e.get("JRT_ANSWER_LENGTH", 50)),
                keep_lead=e.get("JRT_NO_STRIP", "0") == "1", prepend_spaces=int(e.get("JRT_PREPEND_SPACES", "0")))


def recall_prompt(name, doc, tok, keep_lead=None, prepend_spaces=None, **cut):
    """The prompt of one document of recall task `name` (unset options come from `env_options`)."""
    env = env_options()
    keep_lead = env["keep_lead"] if keep_lead is None else keep_lead
    prepend_spaces = env["prepend_spaces"] if prepend_spaces is None else prepend_spaces
    cut.setdefault("context_length", env["context_length"])
    cut.setdefault("answer_length", env["answer_length"])
    _, text_key, answer_keys, kind = RECALL[name]
    d = cut_to_answer(doc, text_key, answer_keys, tok, keep_lead=keep_lead, **cut) or doc
    text = d[text_key]
    lead = text[:len(text) - len(text.lstrip())] if keep_lead else ""
    if kind == "completion":
        return " " * prepend_spaces + (text if keep_lead else text.strip())
    if kind == "extract":
        if name == "swde":
            text = text.split(SUMMARY_MARK)[0]
        text = _strip_question(text, d["key"] + ":")
        body = text.strip("\n").strip().strip("\n").strip().strip(".") if name == "swde" else text.strip("\n").strip(".")
        if not body.endswith("."):
            body += "."
        return lead + body + " " + d["key"][0].upper() + d["key"][1:] + ":"
    body = text.strip()
    if name == "triviaqa":
        body = re.sub(r"\[PAR\]|\[DOC\]|\[TLE\]", "", body)
    question = d["question"].strip()
    body = _strip_question(body, question)
    return lead + body.strip().strip(".") + ". " + question


def recall_labels(doc):
    return list(doc["answers"]) if "answers" in doc else [doc["value"]]


def run_recall(lm, name, docs, tokenizer, shard_spec=None, dump=None, **prompt_kw):
    """Score recall task `name` on `docs` with `lm.generate_until`.  Returns {"contains", "n"}; `dump`:
    path of a jsonl with one {"prompt_tail", "generation", "labels", "metric"} record per document."""
    docs = shard(docs, shard_spec)
    prompts = [recall_prompt(name, d, tokenizer, **prompt_kw) for d in docs]
    gens = lm.generate_until([(p, dict(GEN_RECALL)) for p in prompts])
    hits = [contains_score(g, recall_labels(d)) for g, d in zip(gens, docs)]
    if dump:
        with open(dump, "w") as f:
            for p, g, d, h in zip(prompts, gens, docs, hits):
                f.write(json.dumps({"prompt_tail": p[-200:], "generation": g, "labels": recall_labels(d),
                                    "metric": {"contains": h}}) + "\n")
    return {"contains": sum(hits) / max(1, len(hits)), "n": len(hits)}


# ---- needle tasks ----------------------------------------------------------------------------------
def load_needles(root, task, lengths=(1024, 2048, 4096, 8192)):
    """Documents of `<root>/<task>_<L>/validation.jsonl` for every length present."""
    docs = []
    for L in lengths:
        p = os.path.join(root, f"{task}_{L}", "validation.jsonl")
        if os.path.exists(p):
            for d in load_jsonl(p):
                docs.append({"input": d["input"].rstrip("\n"), "outputs": d["outputs"],
                             "gen_prefix": d["answer_prefix"].strip(), "max_length": int(L)})
    if not docs:
        raise FileNotFoundError(f"no needle data for {task} at {list(lengths)} under {root}")
    return docs


def match_all(prediction, refs):
    """Share of reference strings present in the prediction (case-insensitive)."""
    return sum(r.lower() in prediction.lower() for r in refs) / max(1, len(refs))


def run_needles(lm, docs, shard_spec=None):
    """{length: mean share of needles found, "n": documents}."""
    docs = shard(docs, shard_spec)
    gens = lm.generate_until([(d["input"] + " " + d["gen_prefix"], dict(GEN_NEEDLE)) for d in docs])
    by_len = {}
    for g, d in zip(gens, docs):
        by_len.setdefault(d["max_length"], []).append(match_all(g, d["outputs"]))
    out = {str(L): sum(v) / len(v) for L, v in sorted(by_len.items())}
    out["n"] = len(docs)
    return out


# ---- optional harness classes ------------------------------------------------------------------------
def harness_tasks(tokenizer):
    """{task name: lm_eval task class} for the recall tasks (needs `lm_eval`); names are `jrt_<name>`."""
    from lm_eval.api.instance import Instance
    from lm_eval.api.task import ConfigurableTask

    def make(name):
        hub = RECALL[name][0]

        class Task(ConfigurableTask):
            VERSION, DATASET_PATH, DATASET_NAME = 0, hub, "default"

            def __init__(self, **kw):
                super().__init__(config={"metadata": {"version": self.VERSION}})

            def has_training_docs(self):
                return False

            def has_validation_docs(self):
                return True

            def has_test_docs(self):
                return False

            def validation_docs(self):
                return shard(list(self.dataset["validation"]))

            def doc_to_text(self, doc):
                return recall_prompt(name, doc, tokenizer)

            def doc_to_target(self, doc):
                return recall_labels(doc)[0]

            def construct_requests(self, doc, ctx, **kw):
                kw.pop("chat_template", None), kw.pop("apply_chat_template", None)
                return [Instance(request_type="generate_until", doc=doc, arguments=(ctx, dict(GEN_RECALL)),
                                 idx=0, **kw)]

            def process_results(self, doc, results):
                return {"contains": contains_score(results[0], recall_labels(doc))}

            def aggregation(self):
                return {"contains": lambda v: sum(v) / max(1, len(v))}

            def higher_is_better(self):
                return {"contains": True}

        Task.__name__ = f"Recall_{name}"
        return Task

    return {f"jrt_{n}": make(n) for n in RECALL}
