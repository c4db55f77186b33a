"""The pre-training program end to end on CPU (one process, mock data): logging, evaluation, checkpoint at an exit
interval, resume at the saved iteration with the learning-rate schedule continuing.  The functional-test layer of the
reference (tests/functional_tests) in miniature."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
        "--max-position-embeddings", "32", "--micro-batch-size", "2", "--global-batch-size", "4", "--train-iters", "8",
        "--lr", "1e-3", "--min-lr", "1e-4", "--lr-decay-style", "cosine", "--mock-data", "--tokenizer-type",
        "NullTokenizer", "--vocab-size", "64", "--log-interval", "1", "--eval-interval", "4", "--eval-iters", "2",
        "--save-interval", "4", "--use-cpu-initialization"]


def _run(extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + BASE + extra, capture_output=True,
                       text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    return r.stdout


def _iters(out, loss_key="lm loss"):
    rows = {}
    for m in re.finditer(r"iteration\s+(\d+)/\s*(\d+) .*?learning rate: ([0-9.E+-]+) .*?" + loss_key +
                         r": ([0-9.E+-]+)", out):
        rows[int(m.group(1))] = (float(m.group(3)), float(m.group(4)))
    return rows


def test_train_exit_resume(tmp_path):
    ck = str(tmp_path / "ckpt")
    first = _run(["--save", ck, "--exit-interval", "4"])
    a = _iters(first)
    assert sorted(a) == [1, 2, 3, 4] and "exiting program at iteration 4" in first
    assert "validation loss at iteration 4" in first
    assert open(os.path.join(ck, "latest_checkpointed_iteration.txt")).read().strip() == "4"
    second = _run(["--save", ck, "--load", ck])
    b = _iters(second)
    assert sorted(b) == [5, 6, 7, 8]
    assert b[5][0] < a[4][0] and abs(b[8][0] - 1e-4) < 1e-9            # the cosine schedule carried on to min-lr
    assert "validation loss at iteration 8" in second and "test loss" in second
    # an uninterrupted run reaches the same loss at iteration 8 (same data order, same weights after resume)
    whole = _iters(_run([]))
    assert abs(whole[8][1] - b[8][1]) < 1e-4 and abs(whole[3][1] - a[3][1]) < 1e-6


def test_four_rank_tp2_pp2_program_trains_evaluates_and_saves(tmp_path):
    """torchrun, 4 Gloo ranks, TP2 x PP2 with two virtual stages, sequence parallel, distributed optimizer: the ranks
    that read no data must still take part in evaluation, and every rank writes its checkpoint shard."""
    ck = str(tmp_path / "ckpt")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "pretrain_gpt.py"),
           "--tensor-model-parallel-size", "2", "--pipeline-model-parallel-size", "2",
           "--num-layers-per-virtual-pipeline-stage", "1", "--sequence-parallel", "--use-distributed-optimizer",
           "--distributed-backend", "gloo", "--num-layers", "4", "--hidden-size", "32", "--num-attention-heads", "4",
           "--seq-length", "32", "--max-position-embeddings", "32", "--micro-batch-size", "1", "--global-batch-size", "4",
           "--train-iters", "4", "--lr", "1e-3", "--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64",
           "--log-interval", "1", "--eval-interval", "2", "--eval-iters", "1", "--save", ck, "--save-interval", "4",
           "--use-cpu-initialization", "--attention-dropout", "0", "--hidden-dropout", "0"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert sorted(_iters(out)) == [1, 2, 3, 4]
    assert "validation loss at iteration 2" in out and "validation loss at iteration 4" in out and "test loss" in out
    assert open(os.path.join(ck, "latest_checkpointed_iteration.txt")).read().strip() == "4"
    assert len(os.listdir(os.path.join(ck, "iter_0000004"))) >= 4


def _sentence_corpus(tmp_path):
    import numpy as np
    from megatron_lm_b200.data.indexed_dataset import IndexedDatasetBuilder, get_bin_path, get_idx_path
    prefix = str(tmp_path / "sents")
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    rng = np.random.RandomState(0)
    for _ in range(200):
        for _ in range(rng.randint(3, 7)):
            b.add_item(rng.randint(10, 50, size=rng.randint(4, 12)).tolist())
        b.end_document()
    b.finalize(get_idx_path(prefix))
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(60)]) + "\n")
    return prefix, str(vocab)


def _run_script(script, extra, loss_key="lm loss"):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29618")
    common = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
              "--max-position-embeddings", "64", "--micro-batch-size", "2", "--global-batch-size", "4", "--train-iters",
              "3", "--lr", "1e-3", "--log-interval", "1", "--eval-interval", "2", "--eval-iters", "1",
              "--use-cpu-initialization"]
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)] + common + extra, capture_output=True, text=True,
                       timeout=300, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2500:]
    rows = _iters(out, loss_key)
    assert sorted(rows) == [1, 2, 3] and all(0.5 < v[1] < 10 for v in rows.values()), rows
    assert "validation loss at iteration 2" in out and "test loss" in out
    return out


def test_bert_and_t5_programs_on_a_sentence_corpus(tmp_path):
    prefix, vocab = _sentence_corpus(tmp_path)
    data = ["--data-path", prefix, "--split", "90,5,5", "--tokenizer-type", "BertWordPieceLowerCase", "--vocab-file", vocab]
    out = _run_script("pretrain_bert.py", data)
    assert "sop loss" in out
    out = _run_script("pretrain_t5.py", data + ["--encoder-seq-length", "32", "--decoder-seq-length", "16",
                                                "--vocab-extra-ids", "10", "--encoder-num-layers", "3",
                                                "--decoder-num-layers", "1", "--log-params-norm"])
    assert "params norm" in out


def test_mamba_and_vlm_programs_on_mock_data():
    mock = ["--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64"]
    _run_script("pretrain_mamba.py", mock + ["--mamba-head-dim", "16", "--mamba-num-groups", "2", "--mamba-state-dim", "16"])
    _run_script("pretrain_vlm.py", mock + ["--img-h", "28", "--img-w", "28", "--patch-dim", "14"])


def test_ict_and_vision_classification_programs(tmp_path):
    """The retriever (inverse cloze task, in-batch softmax over pooled BERT embeddings) and the ViT classifier."""
    prefix, vocab = _sentence_corpus(tmp_path)
    out = _run_script("pretrain_ict.py", ["--data-path", prefix, "--split", "90,5,5", "--tokenizer-type",
                                          "BertWordPieceLowerCase", "--vocab-file", vocab, "--retriever-seq-length", "32",
                                          "--retriever-report-topk-accuracies", "1", "2", "--biencoder-projection-dim", "16"],
                      loss_key="retrieval loss")
    assert "top1_acc" in out
    # towers started from a pre-trained BERT checkpoint
    bert_ck = str(tmp_path / "bert_ck")
    data = ["--data-path", prefix, "--split", "90,5,5", "--tokenizer-type", "BertWordPieceLowerCase", "--vocab-file", vocab]
    _run_script("pretrain_bert.py", data + ["--save", bert_ck, "--save-interval", "3"])
    out = _run_script("pretrain_ict.py", data + ["--retriever-seq-length", "32", "--bert-load", bert_ck],
                      loss_key="retrieval loss")
    assert "biencoder towers initialised from the BERT checkpoint" in out
    out = _run_script("pretrain_vision_classify.py", ["--mock-data", "--img-h", "32", "--img-w", "32", "--patch-dim", "8",
                                                      "--num-classes", "4"], loss_key="loss")
    assert "accuracy" in out


def test_ict_blocks_and_samples(tmp_path):
    import numpy as np
    from megatron_lm_b200.data.ict_dataset import ICTDataset, build_blocks_mapping
    from megatron_lm_b200.data.indexed_dataset import IndexedDataset
    prefix, _ = _sentence_corpus(tmp_path)
    ds = IndexedDataset(prefix)
    doc_idx, sizes = np.asarray(ds.document_indices), np.asarray(ds.sequence_lengths)
    m = build_blocks_mapping(doc_idx, sizes, None, 32)
    assert len(m) >= 200 and (m[:, 1] - m[:, 0] >= 2).all()
    for start, end, doc, _ in m[:50]:
        assert doc_idx[doc] <= start < end <= doc_idx[doc + 1]
        assert sizes[start:end].sum() <= 32 - 3 or end - start == 2
    ict = ICTDataset(ds, None, 40, 32, cls_id=2, sep_id=3, pad_id=0, query_in_block_prob=0.0, seed=7)
    s = ict[5]
    q = s["query_tokens"][s["query_pad_mask"] == 1]
    c = s["context_tokens"][s["context_pad_mask"] == 1]
    assert q[0] == 2 and q[-1] == 3 and c[0] == 2 and c[-1] == 3
    start, end = s["block_data"][:2]
    block = [t for i in range(start, end) for t in ds[i]]
    assert len(q) - 2 + len(c) - 2 == len(block)            # the query left its block
    assert np.array_equal(ict[5]["query_tokens"], s["query_tokens"])      # deterministic per index


def _torchrun(nproc, port, extra, script="pretrain_gpt.py"):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, script), "--distributed-backend", "gloo",
           "--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
           "--max-position-embeddings", "32", "--micro-batch-size", "1", "--train-iters", "3", "--lr", "1e-3",
           "--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--log-interval", "1",
           "--eval-interval", "2", "--eval-iters", "1", "--use-cpu-initialization", "--attention-dropout", "0",
           "--hidden-dropout", "0"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert sorted(_iters(out)) == [1, 2, 3] and "validation loss at iteration 2" in out and "test loss" in out
    return out


def test_expert_parallel_and_context_parallel_programs():
    _torchrun(2, 29642, ["--global-batch-size", "4", "--expert-model-parallel-size", "2", "--num-experts", "4",
                         "--moe-router-topk", "2", "--moe-aux-loss-coeff", "0.01", "--moe-router-load-balancing-type",
                         "aux_loss", "--moe-grouped-gemm", "--moe-token-dispatcher-type", "alltoall",
                         "--use-distributed-optimizer"])
    _torchrun(2, 29643, ["--global-batch-size", "2", "--context-parallel-size", "2", "--position-embedding-type", "rope"])


def test_feature_flags_run_in_the_program():
    """Options that change the step's structure: multi-token prediction (modules shared between the main model and
    the prediction heads deliver several gradients per microbatch), full recomputation, the rerun state machine."""
    mock = ["--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64"]
    _run_script("pretrain_gpt.py", mock + ["--mtp-num-layers", "1"])
    _run_script("pretrain_gpt.py", mock + ["--recompute-granularity", "full", "--recompute-method", "uniform",
                                           "--recompute-num-layers", "1", "--rerun-mode", "validate_results"])


def test_sharded_data_parallel_programs_match_replicated_and_resume(tmp_path):
    """--use-custom-fsdp (ZeRO-3 units + sharded AdamW) and --use-torch-fsdp2 train to the same losses as the
    replicated data-parallel path on two ranks, and a custom-FSDP run resumes from its per-rank shard files."""
    base = ["--global-batch-size", "4"]
    ref = _iters(_torchrun(2, 29644, base))
    z3 = _iters(_torchrun(2, 29645, base + ["--use-custom-fsdp", "--data-parallel-sharding-strategy",
                                            "optim_grads_params"]))
    f2 = _iters(_torchrun(2, 29646, base + ["--use-torch-fsdp2"]))
    for it in (1, 2, 3):
        assert abs(ref[it][1] - z3[it][1]) < 1e-5 and abs(ref[it][1] - f2[it][1]) < 1e-5
    ck = str(tmp_path / "ck")
    fs = base + ["--use-custom-fsdp", "--data-parallel-sharding-strategy", "optim_grads_params", "--save", ck,
                 "--save-interval", "2"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    _torchrun(2, 29647, fs)                                      # saves at iteration 2 (and stops at 3)
    assert sorted(os.listdir(os.path.join(ck, "iter_0000002"))) == ["fsdp_rank_00000.pt", "fsdp_rank_00001.pt"]
    with open(os.path.join(ck, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("2")                                               # resume from the mid-run checkpoint
    cmd_tail = fs + ["--load", ck]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29648", os.path.join(ROOT, "pretrain_gpt.py"),
                        "--distributed-backend", "gloo", "--num-layers", "2", "--hidden-size", "32",
                        "--num-attention-heads", "4", "--seq-length", "32", "--max-position-embeddings", "32",
                        "--micro-batch-size", "1", "--train-iters", "3", "--lr", "1e-3", "--mock-data",
                        "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--log-interval", "1",
                        "--eval-interval", "2", "--eval-iters", "1", "--use-cpu-initialization", "--attention-dropout",
                        "0", "--hidden-dropout", "0"] + cmd_tail, capture_output=True, text=True, timeout=280, cwd=ROOT,
                       env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2500:]
    resumed = _iters(out)
    assert sorted(resumed) == [3] and abs(resumed[3][1] - z3[3][1]) < 1e-5


def test_optimizer_cpu_offload_program_matches_the_device_optimizer():
    mock = ["--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--attention-dropout", "0",
            "--hidden-dropout", "0"]
    ref = _iters(_run_script("pretrain_gpt.py", mock))
    for frac in ("1.0", "0.5"):
        got = _iters(_run_script("pretrain_gpt.py", mock + ["--optimizer-cpu-offload", "--optimizer-offload-fraction", frac]))
        assert all(abs(ref[i][1] - got[i][1]) < 1e-5 for i in (1, 2, 3)), (frac, ref, got)


def test_loop_options_on_two_ranks(tmp_path):
    """Options that add collectives or periodic work to the loop must stay in step on every rank: timers written
    to tensorboard (a gather), replica hash checks, manual garbage collection, heartbeat sections; --skip-train
    goes straight to evaluation."""
    tb = str(tmp_path / "tb")
    out = _torchrun(2, 29649, ["--global-batch-size", "4", "--manual-gc", "--manual-gc-interval", "1",
                               "--check-weight-hash-across-dp-replicas-interval", "1", "--enable-ft-package",
                               "--tensorboard-dir", tb, "--log-timers-to-tensorboard", "--log-world-size-to-tensorboard",
                               "--log-validation-ppl-to-tensorboard", "--log-straggler", "--straggler-minmax-count", "2",
                               "--log-progress", "--save", str(tmp_path / "ck"), "--save-interval", "2",
                               "--tensorboard-log-interval", "2", "--log-memory-to-tensorboard"])
    assert "PPL" in out and os.listdir(tb)
    assert "straggler report @ 1" in out and "slowest:" in out
    progress = open(tmp_path / "ck" / "progress.txt").read().splitlines()
    assert sum("Saved checkpoint" in l for l in progress) >= 1 and sum("throughput:" in l for l in progress) == 3
    assert all("# GPUs: 2" in l for l in progress)
    mock = ["--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29619")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + BASE + ["--skip-train"],
                       capture_output=True, text=True, timeout=200, cwd=ROOT, env=env)
    assert r.returncode == 0 and "test loss" in r.stdout and not _iters(r.stdout)


def test_inprocess_restart_after_a_host_side_fault(tmp_path):
    """Rank 1 raises on the host after iteration 3 (first attempt only).  Both ranks abandon the attempt, tear
    their groups down, meet at the store barrier and run again in the same processes, resuming from the latest
    checkpoint; the job still reaches the last iteration and exits 0.  No GPU is involved in the fault."""
    ck = str(tmp_path / "ck")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MLB_INJECT_HOST_FAULT="1:3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29650", os.path.join(ROOT, "pretrain_gpt.py"), "--distributed-backend", "gloo",
           "--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
           "--max-position-embeddings", "32", "--micro-batch-size", "1", "--global-batch-size", "4", "--train-iters", "5",
           "--lr", "1e-3", "--mock-data", "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--log-interval", "1",
           "--eval-interval", "100", "--eval-iters", "0", "--use-cpu-initialization", "--save", ck, "--load", ck,
           "--save-interval", "1", "--inprocess-restart"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=400, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "injected host fault on rank 1 after iteration 3" in out
    assert "[rank 0] in-process restart: attempt 1" in out and "[rank 1] in-process restart: attempt 1" in out
    seen = [int(m.group(1)) for m in re.finditer(r"^ iteration\s+(\d+)/", out, flags=re.M)]
    assert seen[:2] == [1, 2] and seen[-1] == 5 and seen.count(4) == 1


def test_retro_program_builds_its_retrieval_data_and_trains(tmp_path):
    import numpy as np
    from megatron_lm_b200.data.indexed_dataset import IndexedDatasetBuilder, get_bin_path, get_idx_path
    prefix = str(tmp_path / "corpus")
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    rng = np.random.RandomState(0)
    for d in range(24):
        lo = 5 + 4 * (d // 2)
        b.add_item(rng.randint(lo, lo + 8, size=rng.randint(60, 100)).tolist())
        b.end_document()
    b.finalize(get_idx_path(prefix))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29620")
    cmd = [sys.executable, os.path.join(ROOT, "pretrain_retro.py"), "--num-layers", "6", "--hidden-size", "32",
           "--num-attention-heads", "4", "--seq-length", "32", "--max-position-embeddings", "64", "--micro-batch-size", "2",
           "--global-batch-size", "4", "--train-iters", "3", "--lr", "1e-3", "--data-path", prefix, "--split", "90,5,5",
           "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--log-interval", "1", "--eval-interval", "2",
           "--eval-iters", "1", "--use-cpu-initialization", "--retro-chunk-length", "8"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2500:]
    assert sorted(_iters(out)) == [1, 2, 3] and "validation loss at iteration 2" in out and "test loss" in out


def test_pytorch_profiler_window_writes_a_trace(tmp_path):
    tb = str(tmp_path / "tb")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29621")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + BASE +
                       ["--train-iters", "5", "--profile", "--use-pytorch-profiler", "--profile-step-start", "2",
                        "--profile-step-end", "4", "--tensorboard-dir", tb], capture_output=True, text=True, timeout=300,
                       cwd=ROOT, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
    assert any(f.endswith(".pt.trace.json") for f in os.listdir(tb))


def test_injected_result_faults_are_replayed_and_triaged(tmp_path):
    """--error-injection-rate 1 corrupts the first validated loss.  A transient fault is replayed in place and the
    run matches a clean one; a reproducible fault saves the state from before the step and exits with the
    "resume to disambiguate" code, and the restart replays the step and blames the first device."""
    clean = _iters(_run([]))
    out = _run(["--error-injection-rate", "1", "--error-injection-type", "transient_error"])
    assert "result validation, iteration 1: transient_error" in out
    got = _iters(out)
    assert sorted(got) == sorted(clean) and all(abs(got[i][1] - clean[i][1]) < 1e-6 for i in clean)
    ck = str(tmp_path / "ckpt")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + BASE +
                       ["--save", ck, "--error-injection-rate", "1", "--error-injection-type", "persistent_error"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 16, r.stdout[-1500:] + r.stderr[-1500:]
    assert "to replay the step from the checkpoint" in r.stdout and not _iters(r.stdout)
    again = _run(["--save", ck, "--load", ck])
    assert "result validation, iteration 1: persistent_error" in again
    b = _iters(again)
    assert sorted(b) == sorted(clean) and abs(b[8][1] - clean[8][1]) < 1e-4


def test_supervised_finetuning_program_on_a_conversation_file(tmp_path):
    import json
    import random
    rng = random.Random(0)
    path = tmp_path / "chat.jsonl"
    with open(path, "w") as f:
        for _ in range(24):
            turns = []
            for role in ("user", "assistant", "user", "assistant"):
                turns.append({"role": role, "content": " ".join(str(rng.randint(1, 60)) for _ in range(rng.randint(2, 6)))})
            f.write(json.dumps({"messages": turns}) + "\n")
    base = [a for a in BASE if a != "--mock-data"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + base +
                       ["--sft", "--sft-tokenizer-prompt-format", "identity", "--data-path", str(path)],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    rows = _iters(r.stdout)
    assert sorted(rows) == list(range(1, 9)) and rows[8][1] < rows[1][1]
    assert "supervised fine-tuning" in r.stdout and "validation loss at iteration 8" in r.stdout


def test_erasure_coded_checkpoint_over_the_whole_job_without_data_parallelism():
    """TP2 x PP2 on four ranks has one data-parallel replica: the in-memory checkpoint then stripes over all four
    ranks (each contributes its own, different, state) with two parity members per stripe."""
    out = _torchrun(4, 29653, ["--tensor-model-parallel-size", "2", "--pipeline-model-parallel-size", "2",
                               "--global-batch-size", "2", "--non-persistent-ckpt-type", "local",
                               "--non-persistent-save-interval", "2", "--ec-data-shards", "2", "--ec-parity-shards", "2"])
    assert "in-memory erasure-coded checkpoint at iteration 2" in out


_VIT = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "17",
        "--max-position-embeddings", "17", "--micro-batch-size", "4", "--global-batch-size", "8", "--lr", "2e-3",
        "--min-lr", "1e-4", "--lr-decay-style", "cosine", "--mock-data", "--log-interval", "1", "--img-h", "32",
        "--img-w", "32", "--patch-dim", "8", "--num-classes", "4", "--use-cpu-initialization", "--attention-dropout", "0",
        "--hidden-dropout", "0", "--eval-iters", "2"]


def _program(script, extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29655")
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)] + _VIT + extra, capture_output=True, text=True,
                       timeout=280, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_vision_inpainting_program_reconstructs_and_reports_image_metrics():
    out = _program("pretrain_vision_inpaint.py", ["--train-iters", "30", "--eval-interval", "30", "--mask-type", "row",
                                                  "--mask-factor", "1.5"])
    rows = _iters(out, "loss")
    assert sorted(rows)[-1] == 30 and rows[30][1] < 0.6 * rows[1][1]
    assert re.search(r"validation loss at iteration 30 .*psnr value: [0-9.E+-]+ .*ssim value: [0-9.E+-]+", out)


def test_vision_dino_program_trains_with_momentum_teacher_and_knn_monitor():
    out = _program("pretrain_vision_dino.py", ["--train-iters", "12", "--eval-interval", "12", "--dino-out-dim", "64",
                                               "--dino-head-hidden-size", "48", "--dino-bottleneck-size", "16",
                                               "--dino-local-crops-number", "2", "--dino-local-img-size", "16",
                                               "--iter-per-epoch", "4", "--dino-freeze-last-layer", "1",
                                               "--dino-warmup-teacher-temp-epochs", "2", "--knn-bank-size", "32"])
    rows = _iters(out, "loss")
    assert sorted(rows) == list(range(1, 13))
    assert all(0 < v[1] < 6 for v in rows.values())                    # bounded by ln(64) = 4.16 at uniform outputs
    assert re.search(r"validation loss at iteration 12 .*knn_acc_10 value: [0-9.E+-]+", out)


def test_vision_programs_on_the_mit_and_swin_backbones():
    """--vision-backbone-type mit | swin: the classifier and the in-painting model on MiT-B3, DINO towers on Swin."""
    out = _program("pretrain_vision_classify.py", ["--train-iters", "3", "--eval-interval", "3",
                                                   "--vision-backbone-type", "mit"])
    assert "building the mit classification model" in out and sorted(_iters(out, "loss")) == [1, 2, 3]
    assert "accuracy" in out
    out = _program("pretrain_vision_inpaint.py", ["--train-iters", "3", "--eval-interval", "3", "--patch-dim", "4",
                                                  "--vision-backbone-type", "mit"])
    assert sorted(_iters(out, "loss")) == [1, 2, 3] and "psnr value" in out
    out = _program("pretrain_vision_dino.py", ["--train-iters", "3", "--eval-interval", "3", "--dino-out-dim", "64",
                                               "--dino-head-hidden-size", "48", "--dino-bottleneck-size", "16",
                                               "--dino-local-crops-number", "2", "--dino-local-img-size", "16",
                                               "--iter-per-epoch", "4", "--knn-bank-size", "16",
                                               "--vision-backbone-type", "swin", "--swin-backbone-type", "tiny"])
    assert sorted(_iters(out, "loss")) == [1, 2, 3] and "knn_acc_10" in out


def test_moe_run_upcycled_from_a_dense_checkpoint(tmp_path):
    """--moe-use-upcycling: the mixture-of-experts run starts as the dense model (identical experts, top-k weights
    summing to one: the same validation loss), then trains and saves a checkpoint that resumes as a plain MoE run."""
    dense_dir, moe_dir = str(tmp_path / "dense"), str(tmp_path / "moe")
    common = ["--swiglu", "--disable-bias-linear", "--normalization", "RMSNorm", "--ffn-hidden-size", "64",
              "--untie-embeddings-and-output-weights", "--attention-dropout", "0", "--hidden-dropout", "0"]

    def val(out, it):
        m = re.search(rf"validation loss at iteration {it} .*?lm loss value: ([0-9.E+-]+)", out)
        return float(m.group(1))
    dense_out = _run(common + ["--save", dense_dir, "--train-iters", "8", "--save-interval", "8", "--eval-interval", "8"])
    moe_flags = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-aux-loss-coeff", "0", "--moe-grouped-gemm"]
    out = _run(common + moe_flags + ["--moe-use-upcycling", "--load", dense_dir, "--save", moe_dir, "--train-iters", "4",
                                     "--save-interval", "4", "--lr", "1e-9", "--min-lr", "1e-10", "--eval-interval", "1"])
    assert "upcycled the dense checkpoint" in out and "4 expert tensors" in out
    assert sorted(_iters(out)) == [1, 2, 3, 4]
    assert abs(val(out, 1) - val(dense_out, 8)) < 2e-4, (val(out, 1), val(dense_out, 8))
    again = _run(common + moe_flags + ["--load", moe_dir, "--save", moe_dir, "--train-iters", "4", "--lr", "1e-9",
                                       "--min-lr", "1e-10", "--eval-interval", "4"])
    assert "upcycled" not in again
    refused = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_gpt.py")] + BASE + common + moe_flags +
                             ["--moe-use-upcycling", "--load", dense_dir, "--save", moe_dir], capture_output=True,
                             text=True, timeout=200, cwd=ROOT,
                             env=dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29619"))
    assert refused.returncode != 0 and "already holds a checkpoint" in refused.stdout + refused.stderr


def test_checkpoint_format_conversion_and_retained_checkpoints(tmp_path):
    ck, out = str(tmp_path / "ck"), str(tmp_path / "conv")
    _run(["--save", ck, "--save-interval", "2", "--save-retain-interval", "4", "--train-iters", "8", "--exit-interval", "7",
          "--eval-interval", "1000"])
    kept = sorted(d for d in os.listdir(ck) if d.startswith("iter_"))
    assert kept == ["iter_0000004", "iter_0000007"], kept              # multiples of 4 and the newest
    conv = _run(["--load", ck, "--ckpt-convert-format", "torch", "--ckpt-convert-save", out, "--train-iters", "8"])
    assert "converted the checkpoint of iteration 7 to torch" in conv and not _iters(conv)
    assert os.path.isfile(os.path.join(out, "torch", "iter_0000007", "mp_rank_00", "model_optim_rng.pt"))
    resumed = _iters(_run(["--load", os.path.join(out, "torch"), "--train-iters", "8", "--eval-interval", "1000"]))
    again = _iters(_run(["--load", ck, "--train-iters", "8", "--eval-interval", "1000"]))
    assert sorted(resumed) == [8] and abs(resumed[8][1] - again[8][1]) < 1e-5


def test_vision_classifier_head_learning_rate_and_dataset_fractions(tmp_path):
    import numpy as np
    root = tmp_path / "imgs"
    rng = np.random.RandomState(0)
    for split, per in (("train", 6), ("val", 2)):
        for k in range(4):
            d = root / split / f"class{k}"
            d.mkdir(parents=True)
            for i in range(per):
                np.save(d / f"{i}.npy", (rng.rand(3, 32, 32) + 0.5 * k).astype(np.float32))
    sys.path.insert(0, ROOT)
    import pretrain_vision_classify as prog
    ds = prog.ImageFolderDataset(str(root / "train"), 3, 32, 32, 0, classes_fraction=0.5, data_per_class_fraction=0.5)
    assert ds.classes == ["class0", "class1"] and len(ds.items) == 2 * 3
    out = _program("pretrain_vision_classify.py", ["--train-iters", "3", "--eval-interval", "1000", "--head-lr-mult", "10",
                                                   "--data-path", str(root), "--classes-fraction", "0.5"])
    out = out.replace("--mock-data", "")
    assert sorted(_iters(out, "loss")) == [1, 2, 3]


def test_architecture_is_read_back_from_the_checkpoint(tmp_path):
    """--use-checkpoint-args: a run that names only the checkpoint resumes the model that was saved."""
    ck = str(tmp_path / "ck")
    _run(["--save", ck, "--exit-interval", "4", "--swiglu", "--normalization", "RMSNorm", "--disable-bias-linear",
          "--position-embedding-type", "rope", "--untie-embeddings-and-output-weights", "--ffn-hidden-size", "48"])
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29618")
    # wrong sizes on the command line: the stored ones win
    cmd = [sys.executable, os.path.join(ROOT, "pretrain_gpt.py"), "--load", ck, "--use-checkpoint-args", "--num-layers", "5",
           "--hidden-size", "64", "--num-attention-heads", "8", "--micro-batch-size", "2", "--global-batch-size", "4",
           "--train-iters", "8", "--lr", "1e-3", "--min-lr", "1e-4", "--lr-decay-style", "cosine", "--mock-data",
           "--log-interval", "1", "--eval-interval", "1000", "--eval-iters", "0", "--use-cpu-initialization"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert sorted(_iters(r.stdout)) == [5, 6, 7, 8]


def test_hybrid_mamba_program_with_context_parallelism():
    """Two context-parallel ranks: the mixers swap sequence shards for head shards, the attention layer runs the ring."""
    _torchrun(2, 29663, ["--context-parallel-size", "2", "--global-batch-size", "2", "--num-layers", "3",
                         "--mamba-head-dim", "16", "--mamba-num-groups", "2", "--mamba-state-dim", "16",
                         "--hybrid-override-pattern", "M*-", "--position-embedding-type", "rope"],
              script="pretrain_mamba.py")


def test_hybrid_mamba_checkpoint_resumes_under_another_tensor_parallel_size(tmp_path):
    """Saved by two tensor-parallel ranks (distributed optimizer), loaded by one: the mixers' projection and
    convolution segments are re-cut, the test loss of the loaded model is the saved model's."""
    ck = str(tmp_path / "ck")
    model = ["--global-batch-size", "2", "--num-layers", "3", "--mamba-head-dim", "16", "--mamba-num-groups", "2",
             "--mamba-state-dim", "16", "--hybrid-override-pattern", "M*-", "--position-embedding-type", "rope"]
    first = _torchrun(2, 29664, model + ["--tensor-model-parallel-size", "2", "--use-distributed-optimizer", "--save", ck,
                                         "--save-interval", "3"], script="pretrain_mamba.py")

    def test_loss(out):
        return float(re.search(r"test loss \| lm loss value: ([0-9.E+-]+)", out).group(1))

    def resume(train_iters):
        env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29665")
        cmd = [sys.executable, os.path.join(ROOT, "pretrain_mamba.py"), "--distributed-backend", "gloo", "--hidden-size", "32",
               "--num-attention-heads", "4", "--seq-length", "32", "--max-position-embeddings", "32", "--micro-batch-size", "1",
               "--train-iters", str(train_iters), "--lr", "1e-3", "--mock-data", "--tokenizer-type", "NullTokenizer",
               "--vocab-size", "64", "--log-interval", "1", "--eval-interval", "2", "--eval-iters", "1",
               "--use-cpu-initialization", "--attention-dropout", "0", "--hidden-dropout", "0", "--load", ck,
               "--make-vocab-size-divisible-by", "256"] + model      # the padded vocabulary of the two-rank run
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT, env=env)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        return r.stdout
    same = resume(3)                                           # nothing left to train: evaluates the loaded weights
    assert not _iters(same) and abs(test_loss(same) - test_loss(first)) < 2e-4, (test_loss(same), test_loss(first))
