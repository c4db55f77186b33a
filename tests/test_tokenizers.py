"""Tokenizer classes that need model files, built on the fly: WordPiece (vocabulary file, sentinel ids for T5),
SentencePiece (a model trained on a few lines), the Llama-2 flavour, and the factory with vocabulary padding."""
from types import SimpleNamespace

import pytest

from megatron_lm_b200.data.tokenizer import BertWordPieceTokenizer, build_tokenizer


def _vocab(tmp_path):
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "the", "quick", "brown", "fox", "jump", "##s", "##ed", "over",
             "lazy", "dog", ".", ",", "un", "##believ", "##able"]
    p = tmp_path / "vocab.txt"
    p.write_text("\n".join(words) + "\n")
    return str(p), words


def test_wordpiece_greedy_longest_match_and_special_ids(tmp_path):
    path, words = _vocab(tmp_path)
    t = BertWordPieceTokenizer(path, lower_case=True, vocab_extra_ids=3)
    ids = t.tokenize("The quick brown fox jumps over the lazy dog.")
    assert [t.inv[i] for i in ids] == ["the", "quick", "brown", "fox", "jump", "##s", "over", "the", "lazy", "dog", "."]
    assert t.detokenize(ids) == "the quick brown fox jumps over the lazy dog ."
    assert [t.inv[i] for i in t.tokenize("Unbelievable, jumped")] == ["un", "##believ", "##able", ",", "jump", "##ed"]
    assert t.tokenize("zebra") == [t.vocab["[UNK]"]]
    assert (t.pad, t.cls, t.sep, t.mask) == (0, 2, 3, 4)
    assert len(t.additional_special_tokens_ids) == 3 and t.vocab_size == len(words) + 3 + 2
    assert t.bos != t.eos and t.eod == t.eos
    cased = BertWordPieceTokenizer(path, lower_case=False)
    assert cased.tokenize("The") == [cased.vocab["[UNK]"]]            # no lower-casing: not in the vocabulary


def test_sentencepiece_and_llama2(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    from megatron_lm_b200.data.tokenizer import Llama2Tokenizer, SentencePieceTokenizer
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog", "pack my box with five dozen jugs",
                                 "how vexingly quick daft zebras jump", "sphinx of black quartz judge my vow"] * 20))
    prefix = str(tmp_path / "sp")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=60, model_type="bpe",
                                   bos_id=1, eos_id=2, unk_id=0, pad_id=-1)
    t = SentencePieceTokenizer(prefix + ".model", vocab_extra_ids=4)
    text = "the quick brown fox"
    ids = t.tokenize(text)
    assert ids and t.detokenize(ids) == text
    assert t.vocab_size >= 60 + 4 and len({t.bos, t.eos, t.pad, t.eod}) >= 2
    l2 = Llama2Tokenizer(prefix + ".model")
    with_bos = l2.tokenize(text)
    assert with_bos[0] == l2.bos and l2.tokenize(text, bos=False, eos=True)[-1] == l2.eos
    assert l2.detokenize(with_bos[1:]) == text


def test_factory_pads_the_vocabulary(tmp_path):
    path, words = _vocab(tmp_path)
    args = SimpleNamespace(tokenizer_type="BertWordPieceLowerCase", vocab_file=path, vocab_extra_ids=0, rank=0,
                           make_vocab_size_divisible_by=128, tensor_model_parallel_size=2, padded_vocab_size=None)
    t = build_tokenizer(args)
    assert isinstance(t, BertWordPieceTokenizer)
    assert args.padded_vocab_size == 256 and args.padded_vocab_size >= t.vocab_size      # multiple of 128 * tp
    args2 = SimpleNamespace(tokenizer_type="NullTokenizer", vocab_size=1000, rank=0, make_vocab_size_divisible_by=128,
                            tensor_model_parallel_size=1, padded_vocab_size=None)
    build_tokenizer(args2)
    assert args2.padded_vocab_size == 1024
    with pytest.raises(Exception):
        build_tokenizer(SimpleNamespace(tokenizer_type="NoSuchTokenizer", rank=0, make_vocab_size_divisible_by=128,
                                        tensor_model_parallel_size=1))


def test_huggingface_tokenizer_from_a_local_directory(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from megatron_lm_b200.data.tokenizer import HuggingFaceTokenizer
    vocab = {w: i for i, w in enumerate(["<unk>", "<s>", "</s>", "<pad>", "hello", "world", "again"])}
    tk = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    tk.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tk, unk_token="<unk>", bos_token="<s>",
                                                eos_token="</s>", pad_token="<pad>")
    d = tmp_path / "hf_tok"
    fast.save_pretrained(str(d))
    t = HuggingFaceTokenizer(str(d))
    ids = t.tokenize("hello world again hello")
    assert ids == [4, 5, 6, 4] and t.detokenize(ids) == "hello world again hello"
    assert (t.bos, t.eos, t.pad, t.eod) == (1, 2, 3, 2) and t.vocab_size == 7
    assert t.tokenize("unknownword") == [0]
