"""Command line in the manner of ``mlx-one generate`` (src/mlx_one/cli.py:379-446): the same
option names and meanings, plus what a model without a tokenizer needs (``--token-ids``) and
the random-weights mode (``random-model``)."""

from __future__ import annotations

import json
from dataclasses import asdict

import click


@click.group(help="B200-native inference engine for LFM2 models.")
def main() -> None:
    pass


@main.command("generate", help="Generate a completion for PROMPT with the model folder MODEL.")
@click.argument("model")
@click.argument("prompt")
@click.option("--revision", default=None, help="Hub revision; local folders have none.")
@click.option("--offline", is_flag=True, help="Never fetch a model (always so here).")
@click.option("--cache-dir", default=None, help="Where fetched models would be kept (unused).")
@click.option("--max-tokens", type=click.IntRange(min=1), default=128, show_default=True)
@click.option("--temperature", type=click.FloatRange(min=0), default=0.0, show_default=True)
@click.option("--top-k", type=click.IntRange(min=1))
@click.option("--top-p", type=click.FloatRange(min=0, max=1, min_open=True), default=1.0)
@click.option("--seed", type=int, default=0, show_default=True)
@click.option("--stop", multiple=True, help="Stop string; may be repeated.")
@click.option("--stream", is_flag=True, help="Emit token text as it becomes available.")
@click.option("--json-output", "as_json", is_flag=True)
@click.option("--token-ids", is_flag=True,
              help="PROMPT is a list of token ids (comma or space separated); token ids are "
                   "printed. For model folders without a tokenizer.")
@click.option("--dtype", type=click.Choice(["bfloat16", "float32"]), default="bfloat16",
              show_default=True, help="Execution dtype.")
@click.option("--device", default="cuda:0", show_default=True)
def generate_command(model, prompt, revision, offline, cache_dir, max_tokens, temperature, top_k, top_p, seed, stop, stream,
                     as_json, token_ids, dtype, device) -> None:
    from .engine import Engine
    from .sampling import TextGenerationOptions

    try:
        options = TextGenerationOptions(max_tokens=max_tokens, temperature=temperature,
                                        top_k=top_k, top_p=top_p, seed=seed, stop=stop)
        engine = Engine(model, execution_dtype=dtype, device=device, revision=revision,
                        offline=True, cache_dir=cache_dir)
        ids = ([int(v) for v in prompt.replace(",", " ").split()] if token_ids
               else engine.encode(prompt))
        if stream:
            for chunk in engine.stream_ids(ids, options):
                if as_json:
                    click.echo(json.dumps(asdict(chunk), sort_keys=True))
                elif token_ids and chunk.token_id is not None:
                    click.echo(f"{chunk.token_id} ", nl=False)
                elif chunk.text:
                    click.echo(chunk.text, nl=False)
            if not as_json:
                click.echo()
            return
        handle = engine.submit_ids(ids, options, prompt_text="" if token_ids else prompt)
        result = handle.result()
    except (OSError, RuntimeError, ValueError, KeyError) as exc:
        raise click.ClickException(str(exc)) from exc
    if as_json:
        click.echo(result.to_json())
    elif token_ids:
        click.echo(" ".join(str(t) for t in result.token_ids))
    else:
        click.echo(result.text)


@main.command("random-model", help="Write a model folder with random weights from a config.json.")
@click.argument("config", type=click.Path(exists=True, dir_okay=False))
@click.argument("folder", type=click.Path(file_okay=False))
@click.option("--seed", type=int, default=0, show_default=True)
@click.option("--dtype", type=click.Choice(["bfloat16", "float32"]), default="bfloat16")
def random_model_command(config, folder, seed, dtype) -> None:
    import torch

    from .weights import write_random_model

    with open(config) as handle:
        data = json.load(handle)
    try:
        out = write_random_model(folder, data, seed,
                                 torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    except (OSError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(str(out))


if __name__ == "__main__":
    main()
