"""Named corpora for ``prepare_data.py`` (``tools/datasets/corpora.py`` of the reference): download the raw files
(when the machine has network access), then tokenise them with ``preprocess_data``.  A local file can be
registered with ``LocalCorpus`` so the same flow works offline."""
from __future__ import annotations

import os
from abc import ABC, abstractmethod

GPT2_VOCAB_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-vocab.json"
GPT2_MERGE_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-merges.txt"


class DataDownloader(ABC):
    def __init__(self, tokenizer_type=None, merge_file=None, vocab_file=None, data_dir=None, force_redownload=None,
                 num_workers=None):
        self._tokenizer_type = tokenizer_type or "GPT2BPETokenizer"
        self._data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
        self._merge_file = merge_file or (f"{self._data_dir}/gpt2-merges.txt" if self._tokenizer_type == "GPT2BPETokenizer" else None)
        self._vocab_file = vocab_file or {"GPT2BPETokenizer": f"{self._data_dir}/gpt2-vocab.json",
                                          "HFTokenizer": f"{self._data_dir}/20B_tokenizer.json"}.get(self._tokenizer_type)
        self._force_redownload = bool(force_redownload)
        self._num_workers = num_workers or os.cpu_count() or 1

    @property
    def base_dir(self):
        return self._data_dir

    @property
    @abstractmethod
    def name(self):
        ...

    @property
    @abstractmethod
    def urls(self):
        ...

    @property
    def ftfy(self):
        return False

    def exists(self):
        return os.path.isfile(os.path.join(self.base_dir, self.name, self.name + "_text_document.bin"))

    def download(self):
        os.makedirs(os.path.join(self.base_dir, self.name), exist_ok=True)
        for url in self.urls:
            dst = os.path.join(self.base_dir, self.name, os.path.basename(url))
            if not os.path.isfile(dst) or self._force_redownload:
                rc = os.system(f"wget {url} -O {dst}")
                if rc != 0:
                    raise RuntimeError(f"could not download {url} (no network?)")

    def tokenize(self):
        from . import preprocess_data
        parent = os.path.join(self.base_dir, self.name)
        files = ",".join(os.path.join(parent, os.path.basename(u)) for u in self.urls)
        argv = ["--input", files, "--output-prefix", os.path.join(parent, self.name), "--tokenizer-type",
                self._tokenizer_type, "--dataset-impl", "mmap", "--append-eod", "--workers", str(self._num_workers)]
        if self._vocab_file:
            argv += ["--vocab-file", self._vocab_file]
        if self._merge_file:
            argv += ["--merge-file", self._merge_file]
        if self.ftfy:
            argv.append("--ftfy")
        preprocess_data.main(argv)

    def prepare(self):
        if self._force_redownload or not self.exists():
            self.download()
            self.tokenize()


class Enwik8(DataDownloader):
    name = "enwik8"
    urls = ["https://data.deepai.org/enwik8.zip"]


class PileSubset(DataDownloader):
    name = "pile_00"
    urls = ["https://the-eye.eu/public/AI/pile/train/00.jsonl.zst"]


class Pile(DataDownloader):
    name = "pile"
    urls = [f"https://the-eye.eu/public/AI/pile/train/{i:02}.jsonl.zst" for i in range(30)]


class Github(DataDownloader):
    name = "github"
    urls = ["http://eaidata.bmk.sh/data/github_small.jsonl.zst"]


class ArXiv(DataDownloader):
    name = "arxiv"
    urls = ["https://the-eye.eu/public/AI/pile_preliminary_components/2020-09-08-arxiv-extracts-nofallback-until-2007-068.tar.gz"]


class OpenWebText2(DataDownloader):
    name = "openwebtext2"
    urls = ["https://huggingface.co/datasets/segyges/OpenWebText2/resolve/main/openwebtext2.jsonl.zst.tar"]


class C4(DataDownloader):
    name = "c4"
    urls = [f"https://the-eye.eu/eleuther_staging/c4/en/c4-train.{i:05}-of-01024.json.gz" for i in range(1024)]


class LocalCorpus(DataDownloader):
    """An already-present file; ``download`` is a no-op."""

    def __init__(self, name, path, **kw):
        super().__init__(**kw)
        self._name, self._path = name, path

    @property
    def name(self):
        return self._name

    @property
    def urls(self):
        return [self._path]

    def download(self):
        os.makedirs(os.path.join(self.base_dir, self.name), exist_ok=True)
        dst = os.path.join(self.base_dir, self.name, os.path.basename(self._path))
        if os.path.abspath(dst) != os.path.abspath(self._path) and not os.path.exists(dst):
            os.symlink(os.path.abspath(self._path), dst)


DATA_DOWNLOADERS = {"pass": "pass", "enwik8": Enwik8, "pile_subset": PileSubset, "pile": Pile, "github": Github,
                    "arxiv": ArXiv, "openwebtext2": OpenWebText2, "c4": C4}


def prepare_dataset(dataset_name, tokenizer_type=None, data_dir=None, vocab_file=None, merge_file=None,
                    force_redownload=None, num_workers=None):
    data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
    os.makedirs(data_dir, exist_ok=True)
    cls = DATA_DOWNLOADERS.get(dataset_name.lower())
    if cls is None:
        raise NotImplementedError(f'Dataset "{dataset_name}" not recognized - please choose from {list(DATA_DOWNLOADERS)}')
    if cls == "pass":
        return
    cls(tokenizer_type=tokenizer_type, vocab_file=vocab_file, merge_file=merge_file, data_dir=data_dir,
        force_redownload=force_redownload, num_workers=num_workers).prepare()
