"""Benchmark harness on the CPU: matrix construction, command lines, output scraping, one real tiny run, tables."""
import json
import os
import subprocess

import pandas as pd
import pytest
import yaml

from fms_acceleration_b200.benchmarks import benchmark as B
from fms_acceleration_b200.benchmarks import compare_with_reference as CMP
from fms_acceleration_b200.benchmarks import data_processing as DP
from fms_acceleration_b200.benchmarks import display_bench_results as DISP

HERE = os.path.dirname(os.path.abspath(B.__file__))


@pytest.mark.parametrize("fname", ["scenarios.yaml", "scenarios-orca.yaml", "scenarios-moe.yaml",
                                   "scenarios-granite.yaml", "scenarios-liger.yaml"])
def test_shipped_scenarios_reference_known_configs_and_models(fname):
    from fms_acceleration_b200.models.builder import resolve_config

    files = B.framework_config_files()
    for sc in B.load_scenarios(os.path.join(HERE, fname)):
        for fc in sc.framework_configs:
            assert fc is None or (fc in files and os.path.exists(files[fc])), fc
        for args in sc.argument_sets():
            resolve_config(args["model_name_or_path"])


def test_matrix_and_command_lines(tmp_path):
    sc = B.Scenario("s", [None, "accelerated-peft-bnb-foak"],
                    {"model_name_or_path": ["tiny-llama", "tiny-mixtral"], "target_modules": ["q_proj", "v_proj"],
                     "learning_rate": 1e-4})
    exps = B.build_experiments([sc], {"max_steps": 3, "gradient_accumulation_steps": 1}, [1, 2], [4, 6], str(tmp_path),
                               B.framework_config_files())
    assert len(exps) == 2 * 2 * 2 * 2
    e = [x for x in exps if x.num_gpus == 2 and x.framework_config and x.arguments["model_name_or_path"] == "tiny-mixtral"
         and x.arguments["per_device_train_batch_size"] == 3][0]
    argv = e.argv()
    assert argv[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and "--nproc-per-node=2" in argv
    assert argv[argv.index("--master-addr") + 1] == "127.0.0.1"
    i = argv.index("--target_modules")
    assert argv[i + 1:i + 3] == ["q_proj", "v_proj"]
    env = e.environment()
    assert env["CUDA_VISIBLE_DEVICES"] == "0,1" and env[B.ENV_CONFIG].endswith("sample-configuration.yaml")
    e.run(dry_run=True)
    assert "torch.distributed.run" in open(e.path(B.FILE_COMMAND)).read()
    assert json.load(open(e.path(B.FILE_ARGS)))["framework_config"] == "accelerated-peft-bnb-foak"
    # 5 cannot be split over 2 GPUs
    assert all(x.num_gpus == 1 for x in B.build_experiments([sc], {}, [1, 2], [5], str(tmp_path), B.framework_config_files()))
    # a short name without a sample configuration drops out of the matrix
    assert B.build_experiments([B.Scenario("x", ["nope"], {"model_name_or_path": "tiny-llama"})], {}, [1], [4],
                               str(tmp_path), B.framework_config_files()) == []


def test_output_scraping(tmp_path):
    so = tmp_path / "stdout"
    so.write_text("noise\n{'loss': 2.5, 'learning_rate': 1e-4, 'epoch': 0.1}\n{'loss': 2.25, 'epoch': 0.2}\n"
                  "{'train_runtime': 10.0, 'train_tokens_per_second': 1234.5, 'train_loss': 2.3}\n{not a dict}\n")
    res = B.parse_stdout(str(so))
    assert res["train_tokens_per_second"] == 1234.5 and res["loss_trace"] == [2.5, 2.25]
    se = tmp_path / "stderr"
    se.write_text("warning\nTraceback (most recent call last):\n  File \"x.py\", line 1\nValueError: boom\n"
                  "Traceback (most recent call last):\n  File \"y\"\n"
                  "torch.distributed.elastic.multiprocessing.errors.ChildFailedError: \n")
    tb = B.extract_tracebacks(str(se))
    assert len(tb) == 1 and tb[0].strip().endswith("ValueError: boom")
    mem = tmp_path / "mem.csv"
    mem.write_text("timestamp, name, index, memory.used [MiB]\nt, NVIDIA B200, 0, 100 MiB\nt, NVIDIA B200, 0, 300 MiB\n"
                   "t, NVIDIA B200, 1, 200 MiB\n")
    assert B.memory_metrics(str(mem)) == {"mem_nvidia_mem_reserved": 250.0, "gpu_device_name": "NVIDIA B200"}


def test_end_to_end_tiny_run_and_tables(tmp_path):
    scen = tmp_path / "scen.yaml"
    scen.write_text(yaml.safe_dump({"scenarios": [{"name": "lora", "framework_config": [None], "arguments": {
        "model_name_or_path": ["tiny-llama"], "peft_method": "lora", "r": 4, "target_modules": ["q_proj", "v_proj"],
        "max_seq_length": 64, "learning_rate": [1e-3, 2e-3]}}]}))
    out = tmp_path / "results"
    rc = B.main(["--scenarios_config_path", str(scen), "--defaults_config_path", os.path.join(HERE, "defaults.yaml"),
                 "--results_output_path", str(out), "--max_steps", "4", "--effective_batch_size_matrix", "2"])
    assert rc == 0
    summary = pd.read_csv(out / B.FILE_SUMMARY)
    assert len(summary) == 2 and (summary["train_tokens_per_second"] > 0).all()
    assert json.load(open(out / "exp_0" / B.FILE_RESULTS))["train_loss"] > 0
    # a second pass keeps finished experiments
    before = os.path.getmtime(out / "exp_0" / B.FILE_RESULTS)
    B.main(["--scenarios_config_path", str(scen), "--results_output_path", str(out), "--max_steps", "4",
            "--effective_batch_size_matrix", "2", "--no_overwrite"])
    assert os.path.getmtime(out / "exp_0" / B.FILE_RESULTS) == before
    assert DISP.main([str(out), "--keep_columns", "model_name_or_path"]) == 0
    table = pd.read_csv(out / "benchmarks.csv")
    assert "learning_rate" in table.columns and "model_name_or_path" in table.columns and "r" not in table.columns
    # regression check against itself (no outliers), then against a table that is 2x slower
    ref = table.copy()
    ref.to_csv(tmp_path / "ref.csv", index=False)
    args = ["--result_dir", str(out), "--indices", "framework_config", "learning_rate", "--plot_columns",
            "train_tokens_per_second", "train_loss"]
    assert CMP.main(args + ["--reference_benchmark_filepath", str(tmp_path / "ref.csv")]) == 0
    ref["train_tokens_per_second"] *= 0.5
    ref.to_csv(tmp_path / "ref2.csv", index=False)
    assert CMP.main(args + ["--reference_benchmark_filepath", str(tmp_path / "ref2.csv")]) == 1
    assert len(pd.read_csv(out / "outliers.csv")) == 2


def test_data_processing(tmp_path):
    tok = DP.ByteTokenizer()
    rec = {"instruction": "Add.", "input": "1 2", "output": "3"}
    text = DP.build_data_formatting_func(tok)(rec)["output"]
    assert "### Input:\n1 2" in text and text.endswith("### Response: 3<eos>")
    assert "### Input" not in DP.build_data_formatting_func(tok)({"instruction": "Hi", "input": "", "output": "x"})["output"]
    row = DP.build_data_formatting_func(tok, tokenize=True)(rec)
    n_prompt = row["labels"].count(-100)
    assert tok.decode(row["input_ids"][n_prompt:]) == " 3<eos>" and row["labels"][n_prompt:] == row["input_ids"][n_prompt:]
    assert tok.decode(row["input_ids"][:n_prompt]).endswith("### Response:")
    # chat template + separate response field
    tmpl = "Q: {{ messages[0]['instruction'] }}\nA:"
    row = DP.build_data_formatting_func(tok, tokenize=True, chat_template=tmpl, response_template=None,
                                        response_field="output")(rec)
    assert tok.decode(row["input_ids"]) == "Q: Add.\nA:3" and row["labels"][-1] == ord("3") and row["labels"][0] == -100
    with pytest.raises(ValueError):
        DP.build_data_formatting_func(tok, tokenize=True, response_template=None)
    # records without the template are dropped from the cache; the cache is reused
    recs = tmp_path / "r.jsonl"
    recs.write_text("\n".join(json.dumps(r) for r in [rec, rec]))
    path = DP.prepare_dataset(DP.read_records(str(recs)), str(tmp_path / "cache"), "t", tok, max_length=4096)
    rows = json.load(open(path))
    assert len(rows) == 2 and set(rows[0]) == {"input_ids", "labels"}
    assert DP.prepare_dataset([], str(tmp_path / "cache"), "t", tok) == path and len(json.load(open(path))) == 2


def test_shell_driver_dry_run(tmp_path):
    out = tmp_path / "res"
    env = dict(os.environ, DRY_RUN="true")
    r = subprocess.run(["bash", os.path.join(HERE, "run_benchmarks.sh"), "1 2", "4", str(out),
                        os.path.join(HERE, "scenarios-moe.yaml")], env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    cmds = [open(out / d / "command.sh").read() for d in os.listdir(out) if d.startswith("exp_")]
    assert len(cmds) == 24 and any("moe-scattermoe-granite-ep8-foak" in c for c in cmds)


# hub ids that the reference's scenario files name (scripts/benchmarks/scenarios*.yaml)
REFERENCE_SCENARIO_MODELS = [
    "NousResearch/Llama-2-70b-hf", "TheBloke/Llama-2-70B-GPTQ", "TheBloke/Mistral-7B-v0.1-GPTQ",
    "TheBloke/Mixtral-8x7B-Instruct-v0.1-GPTQ", "bigcode/gpt_bigcode-santacoder",
    "ibm-granite/granite-3.0-3b-a800m-instruct", "ibm-granite/granite-4.0-tiny-preview",
    "ibm-research/moe-7b-1b-active-shared-experts", "ibm/PowerLM-3b", "ibm/PowerMoE-3b", "meta-llama/Meta-Llama-3-8B",
    "TechxGenus/Meta-Llama-3-8B-GPTQ", "mistralai/Mistral-7B-v0.1", "mistralai/Mixtral-8x7B-Instruct-v0.1",
]


@pytest.mark.parametrize("hub_id", REFERENCE_SCENARIO_MODELS)
def test_models_of_the_reference_scenarios_resolve_to_presets(hub_id):
    import torch

    from fms_acceleration_b200.models.builder import build_model, resolve_config

    cfg = resolve_config(hub_id)
    with torch.device("meta"):
        model = build_model(cfg, device="meta", dtype=torch.bfloat16)
    billions = sum(p.numel() for p in model.parameters()) / 1e9
    expected = {"Llama-2-70": 69.0, "Mistral-7B": 7.2, "Mixtral-8x7B": 46.7, "santacoder": 1.1, "3b-a800m": 3.3,
                "tiny-preview": 6.7, "7b-1b": 6.4, "PowerLM-3b": 3.5, "PowerMoE-3b": 3.3, "Llama-3-8B": 8.0}
    want = next(v for k, v in expected.items() if k in hub_id)
    assert abs(billions - want) / want < 0.06, (hub_id, billions)


def test_a_scenario_file_in_the_reference_format_runs_through_the_matrix(tmp_path):
    """Hub ids as model names, learning rates written as strings, a framework short name without a sample
    configuration (dropped with a message, as the reference does), the reference's default arguments."""
    scen = {"scenarios": [{"name": "accelerated-peft-bnb",
                           "framework_config": ["accelerated-peft-bnb", "no-such-shortname"],
                           "arguments": {"learning_rate": "2e-4", "torch_dtype": "bfloat16", "peft_method": "lora", "r": 16,
                                         "lora_alpha": 16, "lora_dropout": 0.1,
                                         "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj"],
                                         "model_name_or_path": ["ibm/PowerLM-3b"]}}]}
    defaults = {"use_flash_attn": True, "response_template": "\n### Response:", "dataset_text_field": "output",
                "gradient_checkpointing": True, "evaluation_strategy": "no", "adam_epsilon": "1e-4", "max_steps": 100}
    sp, dp = tmp_path / "scenarios.yaml", tmp_path / "defaults.yaml"
    sp.write_text(yaml.safe_dump(scen))
    dp.write_text(yaml.safe_dump(defaults))
    out = tmp_path / "results"
    rc = B.main(["--num_gpus", "1", "--effective_batch_size_matrix", "4", "--scenarios_config_path", str(sp),
                 "--defaults_config_path", str(dp), "--results_output_path", str(out), "--dry_run"])
    assert rc == 0
    exps = sorted(os.listdir(out))
    assert [e for e in exps if e.startswith("exp_")] == ["exp_0"]  # the unknown short name dropped out
    cmd = (out / "exp_0" / "command.sh").read_text()
    assert "--gradient_checkpointing True" in cmd and "--model_name_or_path ibm/PowerLM-3b" in cmd


def test_trainer_cli_takes_the_reference_default_arguments(capsys):
    from fms_acceleration_b200.benchmarks import sft_trainer as T

    args, unknown = T.build_parser().parse_known_args([
        "--model_name_or_path", "tiny-llama", "--use_flash_attn", "True", "--response_template", "\n### Response:",
        "--dataset_text_field", "output", "--gradient_checkpointing", "True", "--evaluation_strategy", "no",
        "--adam_epsilon", "1e-4", "--include_tokens_per_second", "True", "--save_strategy", "no"])
    assert unknown == [] and args.gradient_checkpointing is True and args.adam_epsilon == 1e-4
    rc = T.main(["--model_name_or_path", "tiny-llama", "--torch_dtype", "float32", "--max_steps", "2", "--logging_steps", "1",
                 "--per_device_train_batch_size", "2", "--max_seq_length", "32", "--gradient_checkpointing", "True",
                 "--gradient_accumulation_steps", "2"])
    assert rc == 0
    text = capsys.readouterr().out
    assert "train_tokens_per_second" in text and "ignored arguments" not in text


def test_runner_options_of_the_reference(tmp_path):
    """Run-wide matrices (sequence lengths, packing), slow scenarios, short name / file pairs, flag aliases."""
    scen = {"scenarios": [
        {"name": "quick", "framework_config": [None, "mine"],
         "arguments": {"model_name_or_path": ["tiny-llama"], "torch_dtype": "float32"}},
        {"name": "heavy", "slow": True, "arguments": {"model_name_or_path": ["tiny-llama"], "packing": False}},
    ]}
    sp = tmp_path / "scenarios.yaml"
    sp.write_text(yaml.safe_dump(scen))
    cfg = tmp_path / "mine.yaml"
    cfg.write_text("plugins: {}\n")
    common = ["--effective_batch_size_matrix", "4", "--scenarios_config_path", str(sp), "--defaults_config_path", "",
              "--dry_run", "--acceleration_framework_config_keypairs", "mine", str(cfg), "--accelerate_config", "unused.yaml",
              "--no_data_processing", "--process_port", "29700", "--preload_models"]
    out = tmp_path / "all"
    assert B.main(["--num_gpus_matrix", "1", "--max_seq_len_matrix", "128", "256", "--packing_matrix", "True",
                   "--results_output_path", str(out)] + common) == 0
    runs = [json.load(open(out / d / B.FILE_ARGS)) for d in sorted(os.listdir(out)) if d.startswith("exp_")]
    # the slow scenario is left out of an unfiltered run; 2 framework settings x 2 sequence lengths remain
    assert len(runs) == 4 and {r["scenario"] for r in runs} == {"quick"}
    assert sorted(r["arguments"]["max_seq_length"] for r in runs) == [128, 128, 256, 256]
    assert all(r["arguments"]["packing"] is True for r in runs)
    assert {r["framework_config"] for r in runs} == {None, "mine"}
    assert any(str(cfg) in open(out / d / B.FILE_COMMAND).read() for d in os.listdir(out) if d.startswith("exp_"))
    # named explicitly, the slow scenario runs; what it fixes itself is not varied
    out2 = tmp_path / "named"
    assert B.main(["--num_gpus", "1", "--packing_matrix", "True", "--run_only_scenarios", "heavy",
                   "--results_output_path", str(out2)] + common) == 0
    runs = [json.load(open(out2 / d / B.FILE_ARGS)) for d in sorted(os.listdir(out2)) if d.startswith("exp_")]
    assert len(runs) == 1 and runs[0]["scenario"] == "heavy" and runs[0]["arguments"]["packing"] is False


def _single_process_sample_configurations():
    import glob

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    names = []
    for f in sorted(glob.glob(os.path.join(here, "sample-configurations", "*-sample-configuration.yaml"))):
        n = os.path.basename(f)[:-len("-sample-configuration.yaml")]
        if not any(t in n for t in ("ep2", "ep4", "ep8", "multipack")):  # those need more than one rank
            names.append((n, f))
    return names


@pytest.mark.parametrize("name,path", _single_process_sample_configurations())
def test_trainer_cli_runs_every_single_process_sample_configuration(name, path, tmp_path, capsys):
    """Two optimizer steps of a tiny model under each sample configuration, with the mixed-precision flag the
    scenario files give (``--bf16 True``, ``--fp16 True`` for GPTQ): loading, augmentation and training go through."""
    from fms_acceleration_b200.benchmarks import sft_trainer as T
    from fms_acceleration_b200.framework import AccelerationFramework
    from fms_acceleration_b200.framework.model_patcher import ModelPatcher

    model = "tiny-granitemoe" if name.startswith("moe-") else "tiny-llama"
    lora = [] if name.startswith(("moe-", "foak-fast", "aadp-")) else ["--peft_method", "lora", "--r", "4", "--lora_alpha", "8"]
    precision = ["--fp16", "True"] if "autogptq" in name else ["--bf16", "True"]
    saved = (dict(ModelPatcher.rules), list(ModelPatcher.history))
    try:
        AccelerationFramework.reset()
        rc = T.main(["--model_name_or_path", model, "--acceleration_framework_config_file", path, "--torch_dtype", "float32",
                     *precision, *lora, "--max_steps", "2", "--logging_steps", "1", "--per_device_train_batch_size", "2",
                     "--max_seq_length", "32", "--output_dir", str(tmp_path)])
    finally:
        AccelerationFramework.reset()
        ModelPatcher.rules.clear()
        ModelPatcher.rules.update(saved[0])
        ModelPatcher.history[:] = saved[1]
    assert rc == 0
    assert "train_tokens_per_second" in capsys.readouterr().out


@pytest.mark.parametrize("name", ["moe-scattermoe-granite-ep2-padding-free-foak", "aadp-padding-free-multipack"])
def test_trainer_cli_runs_two_rank_sample_configurations(name, tmp_path):
    """Expert parallelism of degree 2 and the multipack data loader (which insists on distributed training) on two
    gloo ranks."""
    import sys

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    model = "tiny-granitemoe" if name.startswith("moe-") else "tiny-llama"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29689", "-m", "fms_acceleration_b200.benchmarks.sft_trainer",
           "--model_name_or_path", model, "--acceleration_framework_config_file",
           os.path.join(here, "sample-configurations", f"{name}-sample-configuration.yaml"), "--torch_dtype", "float32",
           "--bf16", "True", "--max_steps", "2", "--logging_steps", "1", "--per_device_train_batch_size", "2",
           "--max_seq_length", "32", "--output_dir", str(tmp_path)]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=here + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=here)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "train_tokens_per_second" in out.stdout


def test_two_rank_lora_experiment_runs_through_the_launcher(tmp_path):
    """A LoRA scenario (``r: 4``) on two ranks, run for real through ``torch.distributed.run`` (gloo on the CPU): the
    rank argument reaches the trainer although the launcher's own parser would take ``--r`` for one of its options."""
    scen = {"scenarios": [{"name": "standard-peft", "arguments": {
        "model_name_or_path": ["tiny-llama"], "torch_dtype": "float32", "bf16": True, "peft_method": "lora", "r": 4,
        "lora_alpha": 8, "lora_dropout": 0.1, "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj"],
        "max_seq_length": 32, "max_steps": 2, "logging_steps": 1}}]}
    sp = tmp_path / "scenarios.yaml"
    sp.write_text(yaml.safe_dump(scen))
    out = tmp_path / "results"
    rc = B.main(["--num_gpus", "2", "--effective_batch_size_matrix", "4", "--scenarios_config_path", str(sp),
                 "--defaults_config_path", "", "--results_output_path", str(out), "--timeout", "600"])
    assert rc == 0
    res = json.load(open(out / "exp_0" / B.FILE_RESULTS))
    assert not res.get("error_messages"), res
    assert res["train_tokens_per_second"] > 0
    assert "--lora_r 4" in open(out / "exp_0" / B.FILE_COMMAND).read()


def test_trainer_cli_on_a_tokenised_file_with_over_long_samples(tmp_path, capsys):
    """Samples longer than ``max_seq_length`` are cut, not dropped (a file of only long samples still trains)."""
    from fms_acceleration_b200.benchmarks import sft_trainer as T

    records = [{"instruction": f"Add {i}", "input": f"{i} + {i + 1}", "output": f"The answer is {2 * i + 1}."}
               for i in range(16)]
    path = DP.prepare_dataset(records, str(tmp_path / "cache"), "bench")
    rows = json.load(open(path))
    assert min(len(r["input_ids"]) for r in rows) > 64
    rc = T.main(["--model_name_or_path", "tiny-llama", "--torch_dtype", "float32", "--training_data_path", path,
                 "--max_steps", "2", "--logging_steps", "1", "--per_device_train_batch_size", "2", "--max_seq_length", "64",
                 "--output_dir", str(tmp_path / "out")])
    assert rc == 0 and "train_tokens_per_second" in capsys.readouterr().out


def test_trainer_cli_saves_and_resumes(tmp_path, capsys):
    """``--save_strategy steps`` writes checkpoints at optimizer-step boundaries and ``--resume_from_checkpoint True``
    continues from the newest one: the resumed run prints the losses of the uninterrupted run."""
    import ast

    from fms_acceleration_b200.benchmarks import sft_trainer as T

    common = ["--model_name_or_path", "tiny-llama", "--torch_dtype", "float32", "--peft_method", "lora", "--r", "4",
              "--lora_alpha", "8", "--logging_steps", "2", "--per_device_train_batch_size", "2", "--max_seq_length", "32",
              "--gradient_accumulation_steps", "2"]

    def losses(argv):
        assert T.main(common + argv) == 0
        lines = [ast.literal_eval(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{'loss'")]
        return [d["loss"] for d in lines]

    whole = losses(["--max_steps", "8", "--output_dir", str(tmp_path / "a")])
    first = losses(["--max_steps", "4", "--save_strategy", "steps", "--save_steps", "2", "--output_dir", str(tmp_path / "b")])
    assert sorted(os.listdir(tmp_path / "b")) == ["checkpoint-2"]  # 4 micro-batches = 2 optimizer steps
    rest = losses(["--max_steps", "8", "--resume_from_checkpoint", "True", "--output_dir", str(tmp_path / "b")])
    assert first == whole[:2] and rest == whole[2:]
    with pytest.raises(ValueError, match="No valid checkpoint"):
        T.main(common + ["--max_steps", "2", "--resume_from_checkpoint", "True", "--output_dir", str(tmp_path / "none")])
