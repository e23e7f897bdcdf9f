"""Native tokenizers: training, exact round trips, persistence, HF byte-level BPE loading."""
import json

from transformers_fusion_b200.tokenizer import BPETokenizer, ByteTokenizer, Qwen35Tokenizer, UnigramTokenizer

CORPUS = ["the quick brown fox jumps over the lazy dog " * 20, "a stitch in time saves nine; the early bird gets the worm " * 20,
          "numbers 12345 and 67890, unicode: naïve café 東京 🙂 " * 10]


def test_bpe_train_roundtrip_save_load(tmp_path):
    t = BPETokenizer().train(CORPUS, 400)
    assert 259 < t.vocab_size <= 400 and t.bos_id == 1 and t.eos_id == 2
    for s in ["the quick brown fox", "naïve café 東京 🙂 12345", "  leading and  double  spaces\n\tok"]:
        ids = t.encode(s)
        assert t.decode(ids) == s
    assert len(t.encode("the quick brown fox")) < len("the quick brown fox")
    t.save(tmp_path / "bpe.txt")
    u = BPETokenizer().load(tmp_path / "bpe.txt")
    assert u.vocab_size == t.vocab_size and u.encode("the lazy dog gets the worm") == t.encode("the lazy dog gets the worm")
    assert t.encode("x", add_bos=True, add_eos=True)[0] == 1


def test_unigram_train_and_tsv(tmp_path):
    t = UnigramTokenizer().train(CORPUS, 300)
    assert t.vocab_size <= 400
    s = "the quick brown fox jumps"
    ids = t.encode(s)
    assert t.decode(ids) == s and len(ids) < len(s)
    t.save(tmp_path / "uni.tsv")
    u = UnigramTokenizer().load(tmp_path / "uni.tsv")
    assert u.encode(s) == ids


def test_hf_byte_level_bpe_and_chat_template(tmp_path):
    # tiny GPT-2 style vocabulary: bytes of "hello world" plus two merges
    t0 = Qwen35Tokenizer()
    alphabet = {}
    for ch in "helowrd":
        alphabet[ch] = len(alphabet)
    alphabet["Ġ"] = len(alphabet)          # the byte-level spelling of " "
    alphabet["he"] = len(alphabet)
    alphabet["hel"] = len(alphabet)
    alphabet["<|endoftext|>"] = len(alphabet)
    (tmp_path / "vocab.json").write_text(json.dumps(alphabet))
    (tmp_path / "merges.txt").write_text("#version: 0.2\nh e\nhe l\n")
    t = Qwen35Tokenizer.load_from_dir(tmp_path)
    ids = t.encode("hello world")
    assert ids[0] == alphabet["hel"] and t.decode(ids) == "hello world"
    assert t.eos_id == alphabet["<|endoftext|>"]
    p = t.apply_chat_template([{"role": "user", "content": "hello"}])
    assert p == "<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n"
    enc = t.encode(p)
    assert t.token_to_id("<|im_start|>") in enc and t.decode(enc).startswith("<|im_start|>")


def test_byte_tokenizer():
    b = ByteTokenizer()
    assert b.decode(b.encode("héllo", add_bos=True, add_eos=True)) == "héllo"
