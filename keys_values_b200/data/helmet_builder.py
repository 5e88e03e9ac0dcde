"""Builds the development / evaluation splits of the HELMET long-context tasks.

Every task yields records ``{"input", "output", "query_id", "max_length"}`` (plus ``qrel`` and
``k_values`` for re-ranking) with the fully formatted HELMET prompt. Sources are the files of
HELMET's ``data.tar.gz`` under ``dataset_parent_dir`` (retrieval, citation, re-ranking and
synthetic recall tasks) or Hugging Face datasets (in-context learning, long-document QA and
summarisation); built splits are cached with ``datasets.DatasetDict.save_to_disk`` next to the
sources in ``<parent>/../longtrain/<task>_<length>`` under the split names ``development`` and
``evaluation``, which is the layout the reference reads and writes
(``keys_values/data/load_helmet_dev_eval.py:197-279``), so caches are interchangeable.

The builder is a table: one :class:`TaskSpec` per dataset key names the family, the prompt
template (HELMET's own prompts; ``get_instruction_template`` returns them with their slots),
the source files per context length and the size of the evaluation split; one function per
family turns source rows into records. Nothing is downloaded implicitly: a missing source
raises ``FileNotFoundError`` with the path (``download_source_data`` fetches the archive when
a network is available).
"""
from __future__ import annotations

import hashlib
import json
import math
import random
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

DATASET_PARENT_DIR = "~/.cache/huggingface/helmet/data"
SOURCE_DATA_URL = "https://huggingface.co/datasets/princeton-nlp/HELMET/resolve/main/data.tar.gz"
LENGTHS = ("8k", "16k", "32k", "64k", "128k")
Record = Dict[str, Any]

_RAG_PROMPT = ("Use the given documents to write a concise and short answer to the question. Write your answer in the following "
               "format:\nAnswer: [answer]\n\n{demos}{context}\n\nQuestion: {question}\nAnswer:")
_CITE_HEAD = ("Instruction: Write an accurate, engaging, and concise answer for the given question using only the provided search "
              "results (some of which might be irrelevant) and cite them properly. Use an unbiased and journalistic tone. Always "
              "cite for any factual claim. When citing a document, surround its ID with square brackets, such as [x] to cite "
              "document x. To cite multiple documents, simply concatenate the citation markers; for example, use [x][y][z] to cite "
              "the documents with ID x, y, and z. Cite at least one document and at most three documents in each sentence. If "
              "multiple documents support the sentence, only cite a minimum sufficient subset of the documents.")
_PROMPTS: Dict[str, Tuple[str, Tuple[str, ...]]] = {
    "rag": (_RAG_PROMPT, ("demos", "context", "question")),
    "cite": ("{demos}" + _CITE_HEAD + "\n\nQuestion: {question}\n\n{context}\n\nAnswer:", ("demos", "question", "context")),
    "rerank": ("You are provided with a list of documents, each indicated by their ID. Rank each document based on their relevance "
               "to the question in descending order from most relelvant to least relevant texts. Include all documents in the "
               "rankings. Write your answer using the unique IDs, with the following format:\nRanking: ID3 > ID1 > ID2\n\n"
               "{demos}{context}\n\nQuery: {question}\nRanking:", ("demos", "context", "question")),
    "icl": ('Use the provided mapping from the text to label to assign a label to the text. Only output "label: {{label}}" and '
            "nothing else. \n\n{context}\n\n{question}\nlabel:", ("context", "question")),
    "narrative_qa": ("You are given a story, which can be either a novel or a movie script, and a question. Answer the question as "
                     "concisely as you can, using a single phrase if possible.\n\n{demos}{context}\n\nQuestion: {question}\nAnswer:",
                     ("demos", "context", "question")),
    "infinite_bench_qa": ("You are given a story and a question. Answer the question as concisely as you can, using a single phrase "
                          "if possible.\n\n{demos}{context}\n\nQuestion: {question}\nAnswer:", ("demos", "context", "question")),
    "infinite_bench_mc": ("You are given a story and a question with multiple choices. Choose the best answer from the options "
                          "provided. Only one of the following options is correct, output the answer using one single letter (A, "
                          "B, C, or D). Don't say anything else.\n\n{demos}{context}\n\nQuestion: {question}\nOptions:\n{options}\n"
                          "Answer:", ("demos", "context", "question", "options")),
    "infinite_bench_sum": ("You are given a book and you are tasked to summarize it. Write a summary of about 1000 to 1200 words. "
                           "Only write about the plot and characters of the story. Do not discuss the themes or background of the "
                           "book. Do not provide any analysis or commentary.\n\n{demos}{context}\n\nNow summarize the book.\n"
                           "Summary:", ("demos", "context")),
    "multi_lex_sum": ("You are given the legal documents in a civil rights lawsuit, and you are tasked to summarize the case. Write "
                      "a concise summary of one paragraph (200 to 250 words). The summary should contain a short description of "
                      "the background, the parties involved, and the outcomes of the case.\n\n{demos}Legal documents:\n{context}\n\n"
                      "Now please summarize the case.\nSummary:", ("demos", "context")),
    "json_kv": ("{context}\n\nExtract the value corresponding to the specified key in the JSON object below.\n\n{demos}Key: "
                "{question}\nCorresponding value:", ("context", "demos", "question")),
    "ruler_one": ("A special magic {type_needle_v} is hidden within the following text. Make sure to memorize it. I will quiz you "
                  "about the {type_needle_v} afterwards.\n{context}\nWhat is the special magic {type_needle_v} for {query} mentioned "
                  "in the provided text?\nThe special magic {type_needle_v} for {query} mentioned in the provided text is",
                  ("type_needle_v", "context", "query")),
    "ruler_many": ("Some special magic {type_needle_v} are hidden within the following text. Make sure to memorize it. I will quiz "
                   "you about the {type_needle_v} afterwards.\n{context}\nWhat are all the special magic {type_needle_v} for {query} "
                   "mentioned in the provided text?\nThe special magic {type_needle_v} for {query} mentioned in the provided text "
                   "are", ("type_needle_v", "context", "query")),
}


def _per_length(pattern: str, counts: Sequence[Any]) -> Dict[str, str]:
    return {length: pattern.format(k=k) for length, k in zip(LENGTHS, counts)}


@dataclass(frozen=True)
class TaskSpec:
    family: str
    prompt: str
    eval_size: int
    files: Dict[str, str] = field(default_factory=dict)   # context length -> source file (relative to the parent dir)
    demo_file: Optional[str] = None
    extra: Dict[str, Any] = field(default_factory=dict)


_K_RAG = (50, 105, 220, 440, 1000)
TASKS: Dict[str, TaskSpec] = {
    "nq": TaskSpec("rag", "rag", 100, _per_length("kilt/nq-dev-multikilt_1000_k{k}_dep6.jsonl", _K_RAG),
                   "kilt/nq-train-multikilt_1000_k3_dep6.jsonl"),
    "trivia_qa": TaskSpec("rag", "rag", 100, _per_length("kilt/triviaqa-dev-multikilt_1000_k{k}_dep6.jsonl", _K_RAG),
                          "kilt/triviaqa-train-multikilt_1000_k3_dep6.jsonl"),
    "hotpot_qa": TaskSpec("rag", "rag", 100, _per_length("kilt/hotpotqa-dev-multikilt_1000_k{k}_dep3.jsonl", _K_RAG),
                          "kilt/hotpotqa-train-multikilt_1000_k3_dep3.jsonl"),
    "pop_qa": TaskSpec("rag", "rag", 100, _per_length("kilt/popqa_test_1000_k{k}_dep6.jsonl", _K_RAG), "kilt/popqa_test_1000_k3_dep6.jsonl",
                       {"id_field": "id", "popularity_log10_below": 3}),
    "alce_asqa": TaskSpec("cite", "cite", 100, {l: "alce/asqa_eval_gtr_top2000.json" for l in LENGTHS}, "alce/prompts/asqa_revised.json",
                          {"num_docs": dict(zip(LENGTHS, (30, 75, 165, 345, 700)))}),
    "alce_qampari": TaskSpec("cite", "cite", 100, {l: "alce/qampari_eval_gtr_top2000.json" for l in LENGTHS},
                             "alce/prompts/qampari_revised.json", {"num_docs": dict(zip(LENGTHS, (30, 75, 165, 345, 700)))}),
    "ms_macro": TaskSpec("rerank", "rerank", 40, _per_length("msmarco/test_reranking_data_k{k}_dep3.jsonl", (50, 130, 285, 600, 1000)),
                         "msmarco/test_reranking_data_k10_dep3.jsonl"),
    "trec_coarse": TaskSpec("icl", "icl", 500, extra={"hub": ("CogComp/trec", None), "label": "coarse_label", "labels": 6,
                                                      "shots": dict(zip(LENGTHS, (400, 800, 1600, 3300, 6600)))}),
    "trec_fine": TaskSpec("icl", "icl", 500, extra={"hub": ("CogComp/trec", None), "label": "fine_label", "labels": 50,
                                                    "shots": dict(zip(LENGTHS, (400, 800, 1600, 3200, 6400)))}),
    "nlu": TaskSpec("icl", "icl", 500, extra={"hub": ("xingkunliuxtracta/nlu_evaluation_data", None), "label": "label", "labels": 68,
                                              "shots": dict(zip(LENGTHS, (510, 1020, 2040, 4080, 8296))), "split_train": 0.1}),
    "banking77": TaskSpec("icl", "icl", 500, extra={"hub": ("PolyAI/banking77", None), "label": "label", "labels": 77,
                                                    "shots": dict(zip(LENGTHS, (360, 720, 1450, 2900, 5900)))}),
    "clinc150": TaskSpec("icl", "icl", 500, extra={"hub": ("clinc_oos", "plus"), "label": "intent", "labels": 151, "test_split": "validation",
                                                   "shots": dict(zip(LENGTHS, (440, 880, 1750, 3525, 7050)))}),
    "narrative_qa": TaskSpec("longdoc", "narrative_qa", 100, extra={"max_tokens": dict(zip(LENGTHS, (7892, 16084, 32468, 65236, 130772)))}),
    "infinite_bench_qa": TaskSpec("longdoc", "infinite_bench_qa", 100,
                                  extra={"config": "longbook_qa_eng", "max_tokens": dict(zip(LENGTHS, (7982, 16174, 32558, 65326, 130862)))}),
    "infinite_bench_mc": TaskSpec("longdoc", "infinite_bench_mc", 100,
                                  extra={"config": "longbook_choice_eng", "max_tokens": dict(zip(LENGTHS, (7982, 16174, 32558, 65326, 130862)))}),
    "infinite_bench_sum": TaskSpec("summ", "infinite_bench_sum", 100,
                                   extra={"config": "longbook_sum_eng", "max_tokens": dict(zip(LENGTHS, (6792, 14984, 31368, 64136, 129672)))}),
    "multi_lex_sum": TaskSpec("summ", "multi_lex_sum", 100, extra={"max_tokens": dict(zip(LENGTHS, (7492, 15684, 32068, 64836, 130372)))}),
    "json_kv": TaskSpec("json_kv", "json_kv", 100, _per_length("json_kv/test_k{k}_dep6.jsonl", (105, 220, 440, 900, 1800))),
    "ruler_mk_needle": TaskSpec("ruler", "ruler_one", 40, _per_length("ruler/niah_multikey_2/validation_{k}.jsonl", (8192, 16384, 32768, 65536, 131072))),
    "ruler_mk_uuid": TaskSpec("ruler", "ruler_one", 40, _per_length("ruler/niah_multikey_3/validation_{k}.jsonl", (8192, 16384, 32768, 65536, 131072))),
    "ruler_mv": TaskSpec("ruler", "ruler_many", 40, _per_length("ruler/niah_multivalue/validation_{k}.jsonl", (8192, 16384, 32768, 65536, 131072))),
}
SUPPORTED_DATASET_KEYS = list(TASKS)


def get_instruction_template(dataset_key: str) -> Tuple[str, Tuple[str, ...]]:
    """``(template, slot names)`` of the task's HELMET prompt."""
    if dataset_key not in TASKS:
        raise KeyError(f"unknown HELMET dataset key {dataset_key!r}; supported: {SUPPORTED_DATASET_KEYS}")
    return _PROMPTS[TASKS[dataset_key].prompt]


# ------------------------------------------------------------------ helpers
def _stable_seed(text: Any) -> int:
    return int(hashlib.sha256(str(text).encode("utf-8")).hexdigest(), 16) % 2**31


def _read_rows(path: Path) -> List[Dict[str, Any]]:
    if not path.is_file():
        raise FileNotFoundError(f"HELMET source file {path} not found (unpack data.tar.gz of princeton-nlp/HELMET there, "
                                f"see download_source_data)")
    text = path.read_text(encoding="utf-8")
    if path.suffix == ".json":
        data = json.loads(text)
        return data if isinstance(data, list) else data.get("data", [data])
    return [json.loads(line) for line in text.splitlines() if line.strip()]


def _first_per_key(rows: List[Dict[str, Any]], key: str) -> List[Dict[str, Any]]:
    seen, out = set(), []
    for r in rows:
        if r[key] not in seen:
            seen.add(r[key])
            out.append(r)
    return out


def _shuffled(rows: List[Any], seed: int) -> List[Any]:
    rows = list(rows)
    random.Random(seed).shuffle(rows)
    return rows


def download_source_data(download_dir: Path) -> None:
    """Fetches and unpacks HELMET's ``data.tar.gz`` into ``download_dir`` (needs a network)."""
    import tarfile
    import tempfile

    import requests

    download_dir = Path(download_dir).expanduser()
    download_dir.mkdir(parents=True, exist_ok=True)
    with tempfile.NamedTemporaryFile(suffix=".tar.gz") as tmp:
        with requests.get(SOURCE_DATA_URL, stream=True, timeout=60) as resp:
            resp.raise_for_status()
            for chunk in resp.iter_content(1 << 20):
                tmp.write(chunk)
        tmp.flush()
        with tarfile.open(tmp.name) as tar:
            tar.extractall(download_dir)


# ----------------------------------------------------------------- families
_PASSAGE = "Document (Title: {title}): {text}"


def _build_rag(key: str, spec: TaskSpec, length: str, parent: Path, **_) -> Tuple[List[Record], List[Record]]:
    rows = _read_rows(parent / spec.files[length])
    demos_all = _read_rows(parent / spec.demo_file)
    qid = spec.extra.get("id_field", "question")
    pool = rows
    if "popularity_log10_below" in spec.extra:  # long-tail entities only in the evaluation split
        pool = [r for r in rows if math.log10(r["s_pop"]) < spec.extra["popularity_log10_below"]]
    chosen = set(random.Random(42).sample(sorted({r[qid] for r in pool}), min(spec.eval_size, len({r[qid] for r in pool}))))
    eval_rows = [r for r in pool if r[qid] in chosen]
    dev_rows = _first_per_key(_shuffled([r for r in rows if r[qid] not in chosen], 42), "question")
    template = _PROMPTS[spec.prompt][0]

    def fill(r: Dict[str, Any]) -> Record:
        cand = [d for d in demos_all if qid == "question" or d[qid] != r[qid]]
        shots = _first_per_key(_shuffled(cand, _stable_seed(r[qid])), qid)[:2]
        demo_text = "".join(
            "\n\n".join(_PASSAGE.format(**c) for c in d["ctxs"]) + f"\n\nQuestion: {d['question']}\nAnswer: {d['answers'][0]}\n\n"
            for d in shots
        )
        context = "\n\n".join(_PASSAGE.format(**c) for c in r["ctxs"])
        return {"input": template.format(demos=demo_text, context=context, question=r["question"]), "output": r["answers"],
                "query_id": r["question"], "max_length": length}

    return [fill(r) for r in dev_rows], [fill(r) for r in eval_rows]


def _build_cite(key: str, spec: TaskSpec, length: str, parent: Path, **_) -> Tuple[List[Record], List[Record]]:
    rows = _read_rows(parent / spec.files[length])
    demo_bank = json.loads((parent / spec.demo_file).read_text(encoding="utf-8"))["demos"]
    n_docs = spec.extra["num_docs"][length]
    doc = "Document [{ID}](Title: {title}): {text}"
    template = _PROMPTS[spec.prompt][0]
    demo_template = _CITE_HEAD + "\n\nQuestion: {question}\n\n{context}\n\nAnswer: {answer}"

    def fill(r: Dict[str, Any]) -> Record:
        context = "\n\n".join(doc.format(ID=i + 1, title=d["title"], text=d["text"]) for i, d in enumerate(r["docs"][:n_docs]))
        shots = random.Random(_stable_seed(r["question"])).sample(demo_bank, 2)
        demos = "\n\n\n".join(
            demo_template.format(question=s["question"], answer=s["answer"],
                                 context="\n\n".join(doc.format(ID=i + 1, title=d["title"], text=d["text"]) for i, d in enumerate(s["docs"])))
            for s in shots
        )
        return {"input": template.format(demos=demos, context=context, question=r["question"]), "output": "", "query_id": r["question"],
                "max_length": length}

    recs = _shuffled([fill(r) for r in rows], 42)
    return recs[spec.eval_size:], recs[: spec.eval_size]


def _build_rerank(key: str, spec: TaskSpec, length: str, parent: Path, **_) -> Tuple[List[Record], List[Record]]:
    rows = _read_rows(parent / spec.files[length])
    demo_rows = _read_rows(parent / spec.demo_file)
    template = _PROMPTS[spec.prompt][0]
    k_values = [k for k in (1, 5, 10, 20, 50, 100, 200, 500, 1000) if k <= len(rows[0]["ctxs"])]

    def passages(ctxs) -> str:
        form = "[ID: {id}] Document (Title: {title}): {text}" if "title" in ctxs[0] else "[ID: {id}] Document: {text}"
        return "\n\n".join(form.format(**c) for c in ctxs)

    def ranking(ctxs) -> str:
        return " > ".join(c["id"] for c in sorted(ctxs, key=lambda c: c["label"], reverse=True))

    def fill(r: Dict[str, Any]) -> Record:
        cand = _first_per_key(_shuffled([d for d in demo_rows if d["qid"] != r["qid"]], _stable_seed(r["qid"])), "qid")[:2]
        demos = "".join(passages(d["ctxs"]) + f"\n\nQuery: {d['query']}\nRanking: {ranking(d['ctxs'])}\n\n" for d in cand)
        return {"input": template.format(demos=demos, context=passages(r["ctxs"]), question=r["query"]), "output": ranking(r["ctxs"]),
                "qrel": [[c["id"], str(c["label"])] for c in r["ctxs"]], "k_values": k_values, "query_id": r["query"], "max_length": length}

    recs = [fill(r) for r in rows]
    return recs[spec.eval_size:], recs[: spec.eval_size]


def _balanced_sample(rows: List[Dict[str, Any]], label_field: str, size: int, seed: int) -> List[Dict[str, Any]]:
    """``size`` rows in rounds that contain every label once (labels with few rows repeat)."""
    rnd = random.Random(seed)
    by_label: Dict[Any, List[Dict[str, Any]]] = {}
    for r in rows:
        by_label.setdefault(r[label_field], []).append(r)
    rounds = math.ceil(size / len(by_label))
    table: List[List[Dict[str, Any]]] = [[] for _ in range(rounds)]
    for samples in by_label.values():
        picks = rnd.sample(range(len(samples)), rounds % len(samples))
        while len(picks) < rounds:
            picks += rnd.sample(range(len(samples)), min(rounds - len(picks), len(samples)))
        for i, idx in enumerate(picks):
            table[i].append(samples[idx])
    for row in table:
        rnd.shuffle(row)
    return [r for row in table for r in row][:size]


def _load_hub(name: str, config: Optional[str]):
    from datasets import load_dataset

    return load_dataset(name, config) if config else load_dataset(name)


def _build_icl(key: str, spec: TaskSpec, length: str, parent: Path, sources: Optional[Dict[str, List[Dict[str, Any]]]] = None,
               **_) -> Tuple[List[Record], List[Record]]:
    """``sources`` may supply ``{"train": rows, "test": rows}`` directly (rows with ``text`` and the label field)."""
    ex = spec.extra
    label = ex["label"]
    if sources is None:
        data = _load_hub(*ex["hub"])
        if "split_train" in ex:
            data = data["train"].train_test_split(test_size=ex["split_train"], seed=42)
        sources = {"train": list(data["train"]), "test": list(data[ex.get("test_split", "test")])}
    train, test = sources["train"], sources["test"]
    template = _PROMPTS[spec.prompt][0]
    n_shots = ex["shots"][length]

    def fill(r: Dict[str, Any], demo_pool: List[Dict[str, Any]]) -> Record:
        seed = (_stable_seed(r["text"]) + 42) % 2**31
        shots = _balanced_sample(demo_pool, label, n_shots, seed)
        names = list(range(ex["labels"]))
        random.Random(seed).shuffle(names)  # labels are renamed per instance, so that they must be read from the context
        context = "\n\n".join(f"{s['text']}\nlabel: {names[int(s[label])]}" for s in shots)
        return {"input": template.format(context=context, question=r["text"]), "output": str(names[int(r[label])]), "query_id": r["text"],
                "max_length": length}

    if key.startswith("trec"):
        held = _shuffled(train, 42)
        dev_src, dev_demos = held[:1000], held[1000:]
        return [fill(r, dev_demos) for r in dev_src], [fill(r, train) for r in test]
    test = _shuffled(test, 42)
    eval_src = _balanced_sample(test, label, spec.eval_size, 42)
    taken = {r["text"] for r in eval_src}
    return [fill(r, train) for r in test if r["text"] not in taken], [fill(r, train) for r in eval_src]


_OMITTED = " ... [the rest of the text is omitted]"


def _truncate_to_tokens(text: str, tokenizer, n_tokens: int) -> str:
    enc = tokenizer(text, return_offsets_mapping=True)
    if len(enc["input_ids"]) <= n_tokens:
        return text
    keep = n_tokens - len(tokenizer(_OMITTED)["input_ids"])
    return text[: enc["offset_mapping"][keep][1]] + _OMITTED


def _build_longdoc(key: str, spec: TaskSpec, length: str, parent: Path, tokenizer=None,
                   sources: Optional[Dict[str, List[Dict[str, Any]]]] = None, **_) -> Tuple[List[Record], List[Record]]:
    """``sources``: ``{"test": rows, "train": rows}`` with ``context, question, answers[, options, id]`` (tests and offline use)."""
    if tokenizer is None:
        raise ValueError(f"HELMET task {key} truncates documents by tokens: a tokenizer must be given")
    budget = spec.extra["max_tokens"][length]
    template = _PROMPTS[spec.prompt][0]
    if key == "narrative_qa":
        if sources is None:
            data = _load_hub("narrativeqa", None)
            sources = {
                "test": [{"context": r["document"]["text"], "question": r["question"]["text"], "answers": [a["text"] for a in r["answers"]]}
                         for r in data["test"].shuffle(seed=42)],
                "train": [{"question": r["question"]["text"], "answers": [a["text"] for a in r["answers"]]} for r in data["train"].select(range(64))],
            }
        rows = [r for r in sources["test"] if len(tokenizer(r["context"])["input_ids"]) >= spec.extra.get("min_tokens", 131072)]
        rnd = random.Random(42)
        recs = []
        for r in rows:
            shots = rnd.sample(sources["train"], 2)
            demos = ("For example:\n\n" + "\n\n".join(f"Question: {s['question']}\nAnswer {s['answers'][0]}" for s in shots)
                     + "\n\nNow, use the following story to answer the question:\n\n")
            recs.append({"input": template.format(demos=demos, context=_truncate_to_tokens(r["context"], tokenizer, budget), question=r["question"]),
                         "output": r["answers"], "query_id": r["question"], "max_length": length})
        return recs[spec.eval_size:], recs[: spec.eval_size]
    # InfiniteBench books: free-form and multiple-choice questions
    if sources is None:
        from datasets import Features, Sequence as Seq, Value, load_dataset

        ft = Features({"id": Value("int64"), "context": Value("string"), "input": Value("string"), "answer": Seq(Value("string")),
                       "options": Seq(Value("string"))})
        sources = {"test": list(load_dataset("xinrongzhang2022/infinitebench", features=ft)[spec.extra["config"]])}
    rows = [dict(r) for r in sources["test"]]
    choice = key.endswith("_mc")
    for r in rows:
        r["question"] = r.get("question", r.get("input"))
        if choice:
            letter = chr(ord("A") + r["options"].index(r["answer"][0]))
            r["answer"] = [letter, f"{letter}. {r['answer'][0]}"]
            r["options_text"] = "A. {}\nB. {}\nC. {}\nD. {}".format(*r["options"])
    demo_form = "[story text]\nQuestion: {q}\n" + ("Options:\n{o}\n" if choice else "") + "Answer: {a}"
    others = _shuffled(rows, 42)

    def demo_block(r) -> str:
        shots = [o for o in others if o["id"] != r["id"]][:2]
        return ("For example:\n\n" + "\n\n".join(demo_form.format(q=s["question"], o=s.get("options_text", ""), a=s["answer"][0]) for s in shots)
                + "\n\nNow, read the following story:")

    rows = _shuffled(rows, 42)
    out: List[Record] = []
    for i, r in enumerate(rows):
        demos = demo_block(r) if i < spec.eval_size else "Now, read the following story:"  # training prompts carry no demonstrations
        out.append({"input": template.format(demos=demos, context=_truncate_to_tokens(r["context"], tokenizer, budget), question=r["question"],
                                             options=r.get("options_text", "")),
                    "output": r["answer"][0], "query_id": r["question"], "max_length": length})
    return out[spec.eval_size:], out[: spec.eval_size]


def _build_summ(key: str, spec: TaskSpec, length: str, parent: Path, tokenizer=None,
                sources: Optional[Dict[str, List[Dict[str, Any]]]] = None, **_) -> Tuple[List[Record], List[Record]]:
    """``sources``: ``{"test": rows, "train": rows}`` with ``context`` and ``summary`` (tests and offline use)."""
    if tokenizer is None:
        raise ValueError(f"HELMET task {key} truncates documents by tokens: a tokenizer must be given")
    budget = spec.extra["max_tokens"][length]
    template = _PROMPTS[spec.prompt][0]
    if sources is None:
        if key == "infinite_bench_sum":
            from datasets import Features, Sequence as Seq, Value, load_dataset

            ft = Features({"id": Value("int64"), "context": Value("string"), "input": Value("string"), "answer": Seq(Value("string")),
                           "options": Seq(Value("string"))})
            rows = [{"context": r["context"], "summary": r["answer"][0]} for r in load_dataset("xinrongzhang2022/infinitebench", features=ft)[spec.extra["config"]]]
            sources = {"test": rows, "train": rows}
        else:
            data = _load_hub("allenai/multi_lexsum", "v20230518")
            conv = lambda r: {"context": "\n\n".join(r["sources"]), "summary": r["summary/short"]}  # noqa: E731
            sources = {"test": [conv(r) for r in data["validation"] if r["summary/short"]],
                       "train": [conv(r) for r in data["train"].select(range(64)) if r["summary/short"]]}
    rows = _shuffled(sources["test"], 42)
    rnd = random.Random(42)
    recs = []
    for r in rows:
        shots = [s for s in rnd.sample(sources["train"], min(3, len(sources["train"]))) if s is not r][:2]
        demos = ("For example:\n\n" + "\n\n".join(f"Summary: {s['summary']}" for s in shots) + "\n\nNow, read the following:\n\n") if shots else ""
        recs.append({"input": template.format(demos=demos, context=_truncate_to_tokens(r["context"], tokenizer, budget)), "output": r["summary"],
                     "query_id": _stable_seed(r["context"][:2000]), "max_length": length})
    return recs[spec.eval_size:], recs[: spec.eval_size]


def _build_json_kv(key: str, spec: TaskSpec, length: str, parent: Path, **_) -> Tuple[List[Record], List[Record]]:
    rows = _read_rows(parent / spec.files[length])
    template = _PROMPTS[spec.prompt][0]
    recs = []
    for r in rows:
        demos = "\n\n".join(f"Key: {k}\nCorresponding value: {v}" for k, v in r["demos"][:2]) + "\n\n"
        recs.append({"input": template.format(context=r["context"], demos=demos, question=r["question"]), "output": r["answer"],
                     "query_id": r["question"], "max_length": length})
    return recs[spec.eval_size:], recs[: spec.eval_size]


def _build_ruler(key: str, spec: TaskSpec, length: str, parent: Path, **_) -> Tuple[List[Record], List[Record]]:
    rows = _read_rows(parent / spec.files[length])
    template = _PROMPTS[spec.prompt][0]
    recs = _shuffled([{"input": template.format(**r), "output": r["outputs"], "query_id": r["query"], "max_length": length} for r in rows], 42)
    return recs[spec.eval_size:], recs[: spec.eval_size]


_FAMILIES: Dict[str, Callable[..., Tuple[List[Record], List[Record]]]] = {
    "rag": _build_rag, "cite": _build_cite, "rerank": _build_rerank, "icl": _build_icl, "longdoc": _build_longdoc, "summ": _build_summ,
    "json_kv": _build_json_kv, "ruler": _build_ruler,
}


def build_helmet_dev_eval(dataset_key: str, max_length: str, dataset_parent_dir: Path, tokenizer=None,
                          sources: Optional[Dict[str, List[Dict[str, Any]]]] = None) -> Tuple[List[Record], List[Record]]:
    """Builds ``(development, evaluation)`` record lists from the sources, without touching the cache."""
    if dataset_key not in TASKS:
        raise ValueError(f"dataset_key = {dataset_key!r} is not supported; choose from {SUPPORTED_DATASET_KEYS}")
    if max_length not in LENGTHS:
        raise ValueError(f"max_length = {max_length!r} must be one of {LENGTHS}")
    spec = TASKS[dataset_key]
    kwargs: Dict[str, Any] = {"tokenizer": tokenizer}
    if sources is not None:
        kwargs["sources"] = sources
    return _FAMILIES[spec.family](dataset_key, spec, max_length, Path(dataset_parent_dir).expanduser(), **kwargs)


def load_helmet_dev_eval(dataset_key: str, tokenizer=None, max_length: str = "8k", dataset_parent_dir: str = DATASET_PARENT_DIR,
                         sources: Optional[Dict[str, List[Dict[str, Any]]]] = None):
    """``(development, evaluation)`` as ``datasets.Dataset`` objects: read from the cache
    ``<parent>/../longtrain/<key>_<length>`` when present, otherwise built and cached there. ``tokenizer`` is a
    ``tokenizers.Tokenizer`` or a Hugging Face fast tokenizer (needed by the tasks that truncate by tokens)."""
    from datasets import Dataset, DatasetDict, load_from_disk

    parent = Path(dataset_parent_dir).expanduser()
    cache_dir = parent.parent / "longtrain" / f"{dataset_key}_{max_length}"
    if cache_dir.is_dir():
        dsd = load_from_disk(str(cache_dir))
        if "development" not in dsd or "evaluation" not in dsd:
            raise ValueError(f"cache at {cache_dir} does not hold the splits 'development' and 'evaluation'")
        return dsd["development"], dsd["evaluation"]
    if tokenizer is not None:
        from tokenizers import Tokenizer as RawTokenizer

        if isinstance(tokenizer, RawTokenizer):  # the tasks that truncate by tokens call it the Hugging Face way
            from transformers import PreTrainedTokenizerFast

            tokenizer = PreTrainedTokenizerFast(tokenizer_object=tokenizer)
    dev, evl = build_helmet_dev_eval(dataset_key, max_length, parent, tokenizer, sources)
    dsd = DatasetDict({"development": Dataset.from_list(dev), "evaluation": Dataset.from_list(evl)})
    cache_dir.parent.mkdir(parents=True, exist_ok=True)
    dsd.save_to_disk(str(cache_dir))
    return dsd["development"], dsd["evaluation"]
