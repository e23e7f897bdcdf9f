"""Streaming client for a Hugging Face style datasets server, plus the small HTTP client it rides on.

``HFStreamer.open(dataset, split)`` pages through ``/rows?dataset=..&config=..&split=..&offset=..&length=..`` of a
datasets-server endpoint and yields the text column of each row; ``HTTPClient`` does plain GET, ranged GET and HEAD with an
optional bearer token.  The endpoint is configurable (``base_url``), so the same client reads a mirror, a local test
server on 127.0.0.1 or - with ``file://`` - a directory of JSON pages; nothing here assumes that the public hub is
reachable.

Reference counterparts: SimpleJSON, HTTPClient (get / range_request / get_content_length / get_binary), HFStreamer
(open / next_sample / close / samples_streamed) - include/quant/hf_streamer.h:22-84, src/trainer/hf_streamer.cpp."""
from __future__ import annotations

import json
import os
import urllib.error
import urllib.parse
import urllib.request
from typing import Iterator, List, Optional


class HTTPClient:
    def __init__(self, timeout_s: float = 30.0):
        self.timeout, self.auth_token = timeout_s, ""

    def set_auth_token(self, token: str): self.auth_token = token

    def _req(self, url: str, method: str = "GET", headers: Optional[dict] = None):
        h = dict(headers or {})
        if self.auth_token:
            h["Authorization"] = f"Bearer {self.auth_token}"
        return urllib.request.urlopen(urllib.request.Request(url, method=method, headers=h), timeout=self.timeout)

    @staticmethod
    def _url(host: str, path: str, https: bool) -> str:
        if "://" in host:
            return host.rstrip("/") + path
        return f"{'https' if https else 'http'}://{host}{path}"

    def get_binary(self, host: str, path: str, https: bool = True) -> bytes:
        with self._req(self._url(host, path, https)) as r:
            return r.read()

    def get(self, host: str, path: str, https: bool = True) -> str:
        return self.get_binary(host, path, https).decode("utf-8", errors="replace")

    def range_request(self, host: str, path: str, start: int, end: int, https: bool = True) -> bytes:
        """Bytes [start, end] inclusive; a server that ignores Range is tolerated (the slice is cut locally)."""
        with self._req(self._url(host, path, https), headers={"Range": f"bytes={start}-{end}"}) as r:
            data = r.read()
            return data if r.status == 206 else data[start:end + 1]

    def get_content_length(self, host: str, path: str, https: bool = True) -> int:
        try:
            with self._req(self._url(host, path, https), method="HEAD") as r:
                return int(r.headers.get("Content-Length", -1))
        except (urllib.error.URLError, ValueError):
            return -1


class SimpleJSON:
    """The handful of extraction helpers the streamer needs, on top of the standard parser."""

    @staticmethod
    def find_array(doc: str, key: str) -> list:
        v = json.loads(doc).get(key, [])
        return v if isinstance(v, list) else []

    @staticmethod
    def find_string(doc: str, key: str) -> str:
        """The first string value stored under ``key`` anywhere in the document (depth first, in document order); "" if none."""
        def walk(v):
            if isinstance(v, dict):
                if isinstance(v.get(key), str):
                    return v[key]
                for c in v.values():
                    r = walk(c)
                    if r is not None:
                        return r
            elif isinstance(v, list):
                for c in v:
                    r = walk(c)
                    if r is not None:
                        return r
            return None
        try:
            return walk(json.loads(doc)) or ""
        except ValueError:
            return ""

    @staticmethod
    def find_all_strings_in_array(arr) -> List[str]:
        """The string elements of a JSON array, given as text or as an already parsed list."""
        if isinstance(arr, str):
            try:
                arr = json.loads(arr)
            except ValueError:
                return []
        return [x for x in arr if isinstance(x, str)] if isinstance(arr, list) else []

    @staticmethod
    def find_object(doc: str, key: str) -> dict:
        v = json.loads(doc).get(key, {})
        return v if isinstance(v, dict) else {}

    @staticmethod
    def find_all_in_array(arr: list, key: str) -> List[str]:
        return [str(x[key]) for x in arr if isinstance(x, dict) and key in x]

    @staticmethod
    def find_all_rfilenames(arr: list) -> List[str]:
        return SimpleJSON.find_all_in_array(arr, "rfilename")

    url_encode = staticmethod(lambda s: urllib.parse.quote(s, safe=""))
    escape = staticmethod(lambda s: json.dumps(s)[1:-1])


class HFStreamer:
    TEXT_KEYS = ("text", "content", "sentence", "document", "code", "question")

    def __init__(self, base_url: str = "https://datasets-server.huggingface.co", page: int = 100, client: Optional[HTTPClient] = None):
        self.base_url, self.page, self.http = base_url.rstrip("/"), page, client or HTTPClient()
        self._open, self._streamed = False, 0
        self._it: Optional[Iterator[str]] = None
        self.dataset = self.split = self.config = ""
        self.last_error = ""

    def is_open(self) -> bool: return self._open
    def samples_streamed(self) -> int: return self._streamed

    def _page_doc(self, offset: int) -> Optional[dict]:
        q = urllib.parse.urlencode({"dataset": self.dataset, "config": self.config, "split": self.split, "offset": offset, "length": self.page})
        try:
            if self.base_url.startswith("file://"):
                p = os.path.join(self.base_url[7:], f"{self.dataset.replace('/', '__')}.{self.split}.{offset}.json")
                if not os.path.exists(p):
                    return None
                return json.load(open(p))
            return json.loads(self.http.get(self.base_url, "/rows?" + q))
        except (urllib.error.URLError, OSError, ValueError) as e:
            self.last_error = str(e)
            return None

    def _rows(self) -> Iterator[str]:
        offset = 0
        while True:
            doc = self._page_doc(offset)
            rows = (doc or {}).get("rows", [])
            if not rows:
                return
            for r in rows:
                row = r.get("row", r) if isinstance(r, dict) else {}
                for k in self.TEXT_KEYS:
                    if isinstance(row.get(k), str):
                        yield row[k]
                        break
                else:
                    s = next((v for v in row.values() if isinstance(v, str)), None)
                    if s is not None:
                        yield s
            offset += len(rows)
            total = (doc or {}).get("num_rows_total")
            if total is not None and offset >= total:
                return

    def open(self, dataset_name: str, split: str = "train", config: str = "default") -> bool:
        self.dataset, self.split, self.config = dataset_name, split, config
        self._streamed, self.last_error = 0, ""
        first = self._page_doc(0)
        self._open = first is not None and "rows" in first
        self._it = self._rows() if self._open else None
        return self._open

    def next_sample(self) -> Optional[str]:
        if not self._open:
            return None
        s = next(self._it, None)
        if s is None:
            return None
        self._streamed += 1
        return s

    def __iter__(self):
        while (s := self.next_sample()) is not None:
            yield s

    def close(self):
        self._open, self._it = False, None
