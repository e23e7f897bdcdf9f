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


def test_unigram_sentencepiece_verbs_and_nbest(tmp_path):
    import math
    t = UnigramTokenizer().train(CORPUS, 300)
    s = "the quick brown fox"
    ids, scores = t.encode_with_scores(s)
    assert ids == t.encode(s) and len(scores) == len(ids) and all(sc <= 0 for sc in scores)
    assert scores == [t.piece_score(i) for i in ids]
    assert UnigramTokenizer.sentencepiece_normalize("  a  b c ") == "▁a▁b▁c"
    assert UnigramTokenizer.sentencepiece_join(["▁the", "▁qu", "ick"]) == "the quick"
    assert t.decode_sentencepiece(ids) == s and t.encode_sentencepiece(s) == ids
    nb = t.encode_nbest(s, 4)
    assert nb[0] == ids and 1 < len(nb) <= 4 and len({tuple(x) for x in nb}) == len(nb)      # best first, all distinct
    total = lambda seg: sum(t.piece_score(i) for i in seg)
    assert all(total(a) >= total(b) - 1e-9 for a, b in zip(nb, nb[1:])) and all(t.decode(x) == s for x in nb)
    assert t.id_to_token(ids[0]).startswith("▁") and t.is_special(0) and not t.is_special(ids[0])
    t.set_unk_id(0), t.set_bos_id(1), t.set_eos_id(2)
    assert (t.unk_id, t.bos_id, t.eos_id) == (0, 1, 2) and t.encode("x", add_bos=True)[0] == 1


def test_wordpiece_tokenizer(tmp_path):
    from transformers_fusion_b200.tokenizer import WordPieceTokenizer
    t = WordPieceTokenizer().train(CORPUS, 120)
    assert t.vocab[:5] == ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] and 40 < t.vocab_size <= 120
    ids = t.encode("the quick brown fox", add_bos=True, add_eos=True)
    assert ids[0] == t.bos_id and ids[-1] == t.eos_id and t.decode(ids) == "the quick brown fox"
    assert any(tok.startswith("##") for tok in t.vocab) and len(t.encode("the")) <= 3
    assert t.encode("xyzzyq§") == [t.unk_id] * 2 or t.unk_id in t.encode("§")          # unseen characters fall back to [UNK]
    t.save(tmp_path / "wp.txt")
    u = WordPieceTokenizer().load(tmp_path / "wp.txt")
    assert u.encode("the lazy dog") == t.encode("the lazy dog") and u.vocab_size == t.vocab_size
    t.set_special_tokens("<unk>", "<s>", "</s>", "<pad>", "<mask>")
    assert t.vocab[:5] == ["<pad>", "<unk>", "<s>", "</s>", "<mask>"] and t.decode(t.encode("the fox", True, True)) == "the fox"


def test_chat_marker_ids(tmp_path):
    alphabet = {ch: i for i, ch in enumerate("helo")}
    alphabet.update({"<|im_start|>": 4, "<|im_end|>": 5, "<|endoftext|>": 6})
    (tmp_path / "vocab.json").write_text(json.dumps(alphabet))
    (tmp_path / "merges.txt").write_text("#version: 0.2\n")
    t = Qwen35Tokenizer.load_from_dir(tmp_path)
    assert t.im_start_id() == 4 and t.im_end_id() == 5 and t.id_to_token(0) == "h"
