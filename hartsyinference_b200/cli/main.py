"""CLI with the reference's verbs for the built modalities: ``text``, ``image``, ``video``,
``embed``, ``serve``, ``convert``, ``models`` / ``list``, ``flags``, ``plan`` (plus an interactive
``chat`` REPL). Placement flags follow src/HartsyInference.Cli/Infra/PlacementCli.cs
(``--gpu``, ``--device "cuda:0+cuda:1"``, ``--parallel auto``) and add the NVSwitch degrees
``--tp / --sp / --ep / --cfg-parallel / --pp``. Multi-GPU runs are SPMD, one process per GPU: a
command whose placement needs N > 1 devices re-launches itself under ``torch.distributed.run`` with
N processes (or is started that way by the user); rank 0 runs the verb, the other ranks follow it.
``--parallel auto`` asks the planner for the placement.
"""
from __future__ import annotations

import json
from pathlib import Path

import click
import torch

from .. import config
from ..engine.requests import EngineOptions, ImageRequest, Modality, ModelSpec, TextRequest, VideoRequest
from ..parallel.config import ParallelConfig


def _engine(device: str, tp: int, sp: int, ep: int, cfg_parallel: bool, pp: int, max_len: int = 8192,
            parallel: str = "", model: str = ""):
    """Build the engine for a verb. Needs-more-than-one-process placements re-launch the command
    under ``torch.distributed.run``; follower ranks serve rank 0 and exit with it."""
    import atexit
    import os
    import subprocess
    import sys
    import torch
    from ..engine.inference_engine import InferenceEngine
    placement = ParallelConfig(tp=tp, sp=sp, ep=max(ep, 1), cfg=2 if cfg_parallel else 1, pp=pp)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if parallel == "auto":
        from ..engine.planner import shape_of_checkpoint, suggest
        gpus = world if world > 1 else (torch.cuda.device_count() if device != "cpu" and torch.cuda.is_available() else 1)
        shape = shape_of_checkpoint(model) if model else None
        if shape is not None and gpus > 1:
            placement = suggest(shape, gpus)
    need = placement.tp * placement.sp * placement.cfg * placement.dp
    if need > 1 and world == 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={need}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29533"),
               "-m", "hartsyinference_b200.cli"] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    eng = InferenceEngine(device, EngineOptions(placement=placement, max_model_len=max_len))
    if not eng.is_front:
        eng.follow()
        sys.exit(0)
    atexit.register(eng.close)          # releases the follower ranks
    return eng


def placement_options(f):
    for opt in (click.option("--device", "--gpu", default="auto", help="auto | cpu | cuda | cuda:N | cuda:0+cuda:1"),
                click.option("--tp", default=1, help="tensor-parallel degree"),
                click.option("--sp", default=1, help="Ulysses sequence-parallel degree (DiT)"),
                click.option("--ep", default=1, help="expert-parallel degree (MoE)"),
                click.option("--cfg-parallel", is_flag=True, help="run the two guidance branches on two device groups"),
                click.option("--pp", default=1, help="pipeline stages (layer / block split)"),
                click.option("--parallel", default="", help="'auto': let the planner choose the placement for the visible GPUs")):
        f = opt(f)
    return f


@click.group()
def cli():
    """hartsyinference-b200: Blackwell-native multimodal inference."""


@cli.command()
@click.argument("model")
@click.argument("prompt")
@click.option("--max-tokens", default=256)
@click.option("--temperature", default=0.7)
@click.option("--top-p", default=0.95)
@click.option("--top-k", default=0)
@click.option("--seed", default=None, type=int)
@click.option("--greedy", is_flag=True)
@click.option("--raw", is_flag=True, help="do not apply the chat template")
@click.option("--json-mode", is_flag=True)
@placement_options
def text(model, prompt, max_tokens, temperature, top_p, top_k, seed, greedy, raw, json_mode, device, tp, sp, ep, cfg_parallel, pp, parallel):
    """Generate text (streams to stdout)."""
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=model)
    req = TextRequest(messages=[] if raw else [{"role": "user", "content": prompt}], prompt=prompt if raw else None,
                      max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k, seed=seed, greedy=greedy,
                      json_mode=json_mode)
    res = None
    for ch in eng.text.stream(ModelSpec(model, Modality.TEXT, local_path=model), req):
        if ch.text:
            click.echo(ch.text, nl=False)
        if ch.result is not None:
            res = ch.result
    click.echo()
    if res is not None:
        click.echo(f"[{res.completion_tokens} tokens, ttft {res.ttft_s * 1e3:.0f} ms, {res.tokens_per_second:.1f} tok/s, {res.stop_reason.value}]", err=True)


@cli.command()
@click.argument("model")
@placement_options
def chat(model, device, tp, sp, ep, cfg_parallel, pp, parallel):
    """Interactive chat REPL (empty line or Ctrl-D quits)."""
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=model)
    spec = ModelSpec(model, Modality.TEXT, local_path=model)
    history: list[dict] = []
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        if not line.strip():
            break
        history.append({"role": "user", "content": line})
        out = ""
        for ch in eng.text.stream(spec, TextRequest(messages=history, max_tokens=1024)):
            if ch.text:
                out += ch.text
                click.echo(ch.text, nl=False)
        click.echo()
        history.append({"role": "assistant", "content": out})


@cli.command()
@click.argument("model")
@click.argument("prompt")
@click.option("--out", "-o", default="out.png")
@click.option("--width", default=1024)
@click.option("--height", default=1024)
@click.option("--steps", default=20)
@click.option("--guidance", default=3.5)
@click.option("--cfg-scale", default=1.0)
@click.option("--negative", default="")
@click.option("--seed", default=None, type=int)
@placement_options
def image(model, prompt, out, width, height, steps, guidance, cfg_scale, negative, seed, device, tp, sp, ep, cfg_parallel, pp, parallel):
    """Generate an image (PNG)."""
    from ..utils.png import encode_png
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=model)
    res = eng.images.generate(ModelSpec(model, Modality.IMAGE, local_path=model if Path(model).exists() else None),
                              ImageRequest(prompt=prompt, negative_prompt=negative, width=width, height=height, steps=steps,
                                           guidance=guidance, cfg_scale=cfg_scale, seed=seed),
                              lambda p: click.echo(f"step {p.step}/{p.total_steps}", err=True))
    Path(out).write_bytes(encode_png(res.rgb, res.width, res.height))
    click.echo(f"{out}: {res.width}x{res.height}, seed {res.seed}, {res.meta.get('step_ms_median', 0):.1f} ms/step")


@cli.command()
@click.argument("model")
@click.argument("prompt")
@click.option("--out-dir", "-o", default="frames")
@click.option("--width", default=832)
@click.option("--height", default=480)
@click.option("--frames", default=81)
@click.option("--steps", default=50)
@click.option("--cfg-scale", default=5.0)
@click.option("--seed", default=None, type=int)
@placement_options
def video(model, prompt, out_dir, width, height, frames, steps, cfg_scale, seed, device, tp, sp, ep, cfg_parallel, pp, parallel):
    """Generate a video (PNG frame sequence; pipe to ffmpeg to mux)."""
    from ..utils.png import encode_png
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=model)
    res = eng.video.generate(ModelSpec(model, Modality.VIDEO, local_path=model if Path(model).exists() else None),
                             VideoRequest(prompt=prompt, width=width, height=height, frames=frames, steps=steps,
                                          cfg_scale=cfg_scale, seed=seed),
                             lambda p: click.echo(f"step {p.step}/{p.total_steps}", err=True))
    d = Path(out_dir)
    d.mkdir(parents=True, exist_ok=True)
    for i, f in enumerate(res.frames):
        (d / f"frame_{i:05d}.png").write_bytes(encode_png(f, res.width, res.height))
    click.echo(f"{len(res.frames)} frames in {d} ({res.width}x{res.height} @ {res.fps} fps)")


@cli.command()
@click.argument("model")
@click.argument("texts", nargs=-1)
@placement_options
def embed(model, texts, device, tp, sp, ep, cfg_parallel, pp, parallel):
    """Embed texts; prints one JSON array per line."""
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=model)
    for e in eng.embeddings.embed(ModelSpec(model, Modality.EMBEDDINGS, local_path=model), list(texts)):
        click.echo(json.dumps([round(float(x), 6) for x in e]))


@cli.command()
@click.argument("model")
@click.argument("wav")
@click.option("--language", default=None, help="two-letter code; detected when omitted")
@click.option("--task", default="transcribe", type=click.Choice(["transcribe", "translate"]))
@click.option("--no-timestamps", is_flag=True)
@click.option("--json", "as_json", is_flag=True, help="print segments as JSON lines")
@click.option("--device", default="auto")
def transcribe(model, wav, language, task, no_timestamps, as_json, device):
    """Speech to text (Whisper checkpoints) from a WAV file."""
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import AudioRequest
    eng = InferenceEngine(device)
    res = eng.transcribe.run(ModelSpec(model, Modality.TRANSCRIBE, local_path=model),
                             AudioRequest(audio=wav, language=language, task=task, timestamps=not no_timestamps))
    if as_json:
        for s in res.segments:
            click.echo(json.dumps({"start": round(s.start, 2), "end": round(s.end, 2), "text": s.text}))
    else:
        click.echo(res.text)


@cli.command()
@click.argument("model")
@click.argument("image")
@click.option("--out", default="upscaled.png")
@click.option("--tile", default=128, help="input-space tile size (0 = whole image)")
@click.option("--device", default="auto")
def restore(model, image, out, tile, device):
    """Upscale an image with a Real-ESRGAN checkpoint."""
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import RestoreRequest
    from ..utils.png import encode_png
    eng = InferenceEngine(device)
    res = eng.restore.run(ModelSpec(model, Modality.RESTORE, local_path=model), RestoreRequest(image=image, tile=tile))
    Path(out).write_bytes(encode_png(res.rgb, res.width, res.height))
    click.echo(f"{out}: {res.width}x{res.height}")


@cli.command(name="3d")
@click.argument("model")
@click.argument("image")
@click.option("--out", default="mesh.glb", help=".obj, .ply or .glb")
@click.option("--resolution", default=256, help="lattice points per axis of the density field")
@click.option("--threshold", default=None, type=float, help="density iso level (model default when omitted)")
@click.option("--device", default="auto")
def mesh3d(model, image, out, resolution, threshold, device):
    """Reconstruct a textured mesh from one image (TripoSR checkpoints)."""
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import MeshRequest
    eng = InferenceEngine(device)
    res = eng.mesh.run(ModelSpec(model, Modality.MESH, local_path=model),
                       MeshRequest(image=image, resolution=resolution, threshold=threshold, output_path=out))
    click.echo(f"{out}: {len(res.vertices)} vertices, {len(res.faces)} faces "
               f"(triplane {res.meta['triplane_s']:.2f} s, field + surface {res.meta['mesh_s']:.2f} s)")


@cli.command()
@click.argument("model")
@click.argument("image")
@click.option("--actions", default=None, help="JSON file: a list of action rows (25 floats each); default: --frames rows of zeros")
@click.option("--frames", default=8, help="frames to generate when no action file is given")
@click.option("--out", default="world_frames", help="directory for frame_NNNN.png")
@click.option("--seed", default=0)
@click.option("--device", default="auto")
def world(model, image, actions, frames, out, seed, device):
    """Play an action-conditioned world model (Oasis checkpoints) from a first picture."""
    import json
    import os
    import torch
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import WorldRequest
    from ..utils.png import encode_png
    rows = json.load(open(actions)) if actions else [[0.0] * 25 for _ in range(frames)]
    eng = InferenceEngine(device)
    res = eng.world.run(ModelSpec(model, Modality.WORLD, local_path=model), WorldRequest(image=image, actions=rows, seed=seed))
    os.makedirs(out, exist_ok=True)
    for i, f in enumerate(res.frames):
        rgb = (f.clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).contiguous()
        with open(os.path.join(out, f"frame_{i:04d}.png"), "wb") as fh:
            fh.write(encode_png(rgb.numpy().tobytes(), rgb.shape[1], rgb.shape[0]))
    click.echo(f"{out}: {len(res.frames)} frames, {res.meta['seconds_per_frame']:.3f} s per generated frame")


@cli.command()
@click.argument("model")
@click.argument("text")
@click.option("--out", default="speech.wav")
@click.option("--speed", default=None, type=float)
@click.option("--device", default="auto")
def speak(model, text, out, speed, device):
    """Text to speech (VITS voices: MMS-TTS / Piper class) into a WAV file."""
    from ..audio import write_wav
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import SpeechRequest
    eng = InferenceEngine(device)
    res = eng.speech.run(ModelSpec(model, Modality.SPEECH, local_path=model), SpeechRequest(text=text, speed=speed))
    write_wav(out, res.samples, res.sample_rate)
    click.echo(f"{out}: {res.seconds:.2f} s at {res.sample_rate} Hz")


@cli.command()
@click.argument("wav")
@click.option("--out", default="fx.wav")
@click.option("--op", "ops_", multiple=True, type=click.Choice(["normalize-peak", "normalize-rms", "trim", "resample", "pitch"]),
              help="applied in the order given")
@click.option("--peak", default=0.95, type=float)
@click.option("--rms", default=0.1, type=float)
@click.option("--rate", default=0, type=int, help="target rate of 'resample'")
@click.option("--silence-db", default=-45.0, type=float, help="'trim': level under which the edges are cut")
def fx(wav, out, ops_, peak, rms, rate, silence_db):
    """Signal-processing effects on a WAV file: level normalisation, silence trimming, resampling, pitch contour
    (the learned effects of the reference, stem separation and speech enhancement, are not built)."""
    from ..audio import read_wav, write_wav
    from ..audio import dsp
    from ..audio.wav import resample
    x, sr = read_wav(wav)
    x = x.mean(0) if x.dim() > 1 else x
    for op in ops_ or ("normalize-peak",):
        if op == "normalize-peak":
            x = dsp.normalize_peak(x, peak)
        elif op == "normalize-rms":
            x = dsp.normalize_rms(x, rms, peak)
        elif op == "resample":
            if rate <= 0:
                raise click.UsageError("'resample' needs --rate")
            x, sr = resample(x, sr, rate), rate
        elif op == "trim":
            frame = max(1, sr // 100)
            level = x[:x.numel() // frame * frame].view(-1, frame).pow(2).mean(1).clamp_min(1e-12).log10() * 10
            loud = (level > silence_db).nonzero().flatten()
            if loud.numel():
                x = x[max(0, (int(loud[0]) - 5) * frame):min(x.numel(), (int(loud[-1]) + 6) * frame)]
        elif op == "pitch":
            x16 = resample(x, sr, 16000) if sr != 16000 else x
            f0 = dsp.estimate_f0(x16, 16000, 320)
            voiced = f0[f0 > 0]
            click.echo(f"pitch: {voiced.numel()}/{f0.numel()} voiced frames" +
                       (f", median {float(voiced.median()):.1f} Hz, range {float(voiced.min()):.1f}-{float(voiced.max()):.1f} Hz" if voiced.numel() else ""))
    write_wav(out, x.clamp(-1, 1), sr)
    click.echo(f"{out}: {x.numel() / sr:.2f} s at {sr} Hz")


@cli.command(name="wake-listen")
@click.argument("models_dir")
@click.option("--host", default="127.0.0.1")
@click.option("--port", "-p", default=10400, type=int)
@click.option("--threshold", default=0.5, type=float)
@click.option("--device", default="cpu")
def wake_listen(models_dir, host, port, threshold, device):
    """Serve wake-word detection to voice satellites (Wyoming protocol). MODELS_DIR holds melspectrogram and
    embedding_model files plus one head per wake word."""
    from ..audio.wake import WakeModelSet, WakeWordSettings
    from ..server.wyoming import WyomingWakeServer
    models = WakeModelSet(models_dir, device)
    click.echo(f"wake words: {', '.join(models.heads) or '(none)'}; listening on {host}:{port}")
    WyomingWakeServer(models, host, port, {n: WakeWordSettings(threshold=threshold) for n in models.heads}).serve_forever()


@cli.command(name="wake-client")
@click.argument("wav")
@click.option("--host", default="127.0.0.1")
@click.option("--port", "-p", default=10400, type=int)
@click.option("--word", "words", multiple=True, help="only these wake words")
@click.option("--realtime", is_flag=True, help="pace the stream like a microphone")
def wake_client(wav, host, port, words, realtime):
    """Stream a WAV file to a wake-word listener as a voice satellite would."""
    import asyncio
    from ..audio import read_wav
    from ..server.wyoming import stream_wav
    samples, rate = read_wav(wav)
    if samples.dim() > 1:
        samples = samples.mean(0)
    hits = asyncio.run(stream_wav(host, port, samples, rate, words or None, realtime=realtime))
    for h in hits:
        click.echo(f"{h['name']} at {h['timestamp'] / 1000:.2f} s (score {h.get('score', 0):.2f})")
    if not hits:
        click.echo("no wake word detected")


@cli.command(name="wake-train")
@click.argument("phrase")
@click.option("--models-dir", required=True, help="directory with melspectrogram / embedding_model; the head is written here")
@click.option("--voice", "voices", multiple=True, required=True, help="text-to-speech checkpoint(s) that say the phrase")
@click.option("--negative-audio", "negative_dirs", multiple=True, help="directories of WAV files that do not hold the phrase")
@click.option("--negative-phrase", "negative_phrases", multiple=True, help="other sentences spoken by the same voices")
@click.option("--epochs", default=40, type=int)
@click.option("--device", default="cpu")
def wake_train(phrase, models_dir, voices, negative_dirs, negative_phrases, epochs, device):
    """Train a new wake word from its text with the engine's own text-to-speech voices."""
    from pathlib import Path
    from ..audio import read_wav
    from ..audio.wake import RATE, WakeModelSet, train_wake_word
    from ..audio.wav import resample
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import SpeechRequest
    eng = InferenceEngine(device)
    models = WakeModelSet(models_dir, device)

    def say(voice, text, speed):
        res = eng.speech.run(ModelSpec(voice, Modality.SPEECH, local_path=voice), SpeechRequest(text=text, speed=speed))
        x = res.samples.float().cpu()
        return (resample(x, res.sample_rate, RATE) if res.sample_rate != RATE else x) * 32767.0

    positives = [say(v, phrase, s) for v in voices for s in (0.85, 1.0, 1.15)]
    others = list(negative_phrases) or ["what time is it", "turn on the kitchen lights please", "the weather looks fine today",
                                        "play some music in the living room", "set a timer for ten minutes"]
    negatives = [torch.cat([say(v, t, 1.0) for t in others]) for v in voices]
    for d in negative_dirs:
        for f in sorted(Path(d).expanduser().glob("**/*.wav")):
            x, rate = read_wav(f)
            x = x.mean(0) if x.dim() > 1 else x
            negatives.append((resample(x, rate, RATE) if rate != RATE else x) * 32767.0)
    name = "_".join(phrase.lower().split())
    report = train_wake_word(models, name, positives, negatives, epochs=epochs, log=click.echo)
    click.echo(f"wrote {report['path']}: recall {report['recall']:.2f}, false accepts {report['false_accepts']:.3f} on the training windows")


@cli.command()
@click.argument("model")
@click.argument("prompt")
@click.option("--out", default="music.wav")
@click.option("--seconds", default=5.0)
@click.option("--guidance", default=3.0)
@click.option("--greedy", is_flag=True)
@click.option("--seed", default=0)
@click.option("--device", default="auto")
def music(model, prompt, out, seconds, guidance, greedy, seed, device):
    """Text to music (MusicGen) into a WAV file."""
    from ..audio import write_wav
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import MusicRequest
    eng = InferenceEngine(device)
    res = eng.music.run(ModelSpec(model, Modality.MUSIC, local_path=model),
                        MusicRequest(prompt=prompt, seconds=seconds, guidance=guidance, greedy=greedy, seed=seed))
    write_wav(out, res.samples, res.sample_rate)
    click.echo(f"{out}: {res.seconds:.2f} s at {res.sample_rate} Hz")


@cli.command()
@click.argument("model")
@click.option("--image", "images", multiple=True, help="image file (repeatable)")
@click.option("--text", "texts", multiple=True, help="caption / query / prompt (repeatable)")
@click.option("--op", "operation", default="embed", type=click.Choice(["embed", "depth", "segment", "detect"]))
@click.option("--threshold", default=0.1, help="score threshold of detect")
@click.option("--device", default="auto")
def vision(model, images, texts, operation, threshold, device):
    """Image embeddings / similarity (CLIP, SigLIP, DINOv2), depth, text-prompted segmentation, open-vocabulary detection."""
    from ..engine.inference_engine import InferenceEngine
    from ..engine.requests import VisionRequest
    eng = InferenceEngine(device)
    res = eng.vision.run(ModelSpec(model, Modality.VISION, local_path=model),
                         VisionRequest(operation=operation, images=list(images), texts=list(texts), score_threshold=threshold))
    if res.detections is not None:
        for img, dets in zip(images, res.detections):
            for dt in dets:
                click.echo(json.dumps({"image": img, **dt}))
        return
    if res.depth is not None or res.masks is not None:
        for img, t in zip(images, res.depth if res.depth is not None else res.masks):
            click.echo(json.dumps({"image": img, "shape": list(t.shape), "min": float(t.min()), "max": float(t.max())}))
        return
    out = res.similarity if res.similarity is not None else (res.image_embeddings if res.image_embeddings is not None else res.text_embeddings)
    for row in (out if out is not None else []):
        click.echo(json.dumps([round(float(x), 6) for x in row]))


@cli.command()
@click.option("--host", default="127.0.0.1")
@click.option("--port", default=8080)
@click.option("--model", "models", multiple=True, help="name=path (repeatable)")
@click.option("--api-key", "api_keys", multiple=True)
@click.option("--max-concurrency", default=1)
@click.option("--max-queue-depth", default=16)
@click.option("--allow-model-paths", is_flag=True, help="let API callers name arbitrary local paths as models")
@placement_options
def serve(host, port, models, api_keys, max_concurrency, max_queue_depth, allow_model_paths, device, tp, sp, ep, cfg_parallel,
          pp, parallel):
    """Run the HTTP server (rank 0 of a multi-GPU placement hosts it; the other ranks follow)."""
    import uvicorn
    from ..server import ServerOptions, create_app
    table = dict(m.split("=", 1) for m in models)
    first = next(iter(table), None)
    eng = _engine(device, tp, sp, ep, cfg_parallel, pp, parallel=parallel, model=table.get(first, "") if first else "")
    app = create_app(ServerOptions(backend=device, models=table, api_keys=list(api_keys), max_concurrency=max_concurrency,
                                   max_queue_depth=max_queue_depth, default_text_model=first,
                                   allow_model_paths=allow_model_paths), engine=eng)
    uvicorn.run(app, host=host, port=port)


@cli.command()
@click.argument("src")
@click.argument("dst")
@click.option("--quant", default=None, help="GGUF target type for 2-D tensors: Q8_0 | Q4_0 | Q4_K")
def convert(src, dst, quant):
    """Convert between checkpoint containers: .safetensors <-> .gguf (optionally quantising), or .pth -> .safetensors."""
    import torch
    from ..assets import gguf as G
    from ..assets.safetensors import SafeTensorsFile, save_file
    if Path(src).is_dir() and dst.endswith(".gguf"):
        # a Hugging Face decoder directory: architecture-aware conversion (names, q/k permutation, experts, tokenizer)
        from ..assets.converters import hf_to_gguf
        md = hf_to_gguf(src, dst, quant)
        click.echo(f"{md['general.architecture']}: {md.get(md['general.architecture'] + '.block_count')} blocks")
    elif src.endswith(".gguf") and dst.endswith(".safetensors"):
        f = G.GgufFile(src)
        save_file({k: f.get(k) for k in f.keys()}, dst, {"format": "pt", "source": Path(src).name})
    elif dst.endswith(".gguf"):
        f = SafeTensorsFile(src)
        G.write_gguf(dst, {"general.name": Path(src).stem}, {k: f.get(k).float() for k in f.keys()},
                     quant=G.GGML_TYPES[quant] if quant else None)
    elif src.endswith((".pth", ".pt", ".bin")):
        sd = torch.load(src, map_location="cpu", weights_only=True)
        sd = sd.get("state_dict", sd) if isinstance(sd, dict) else sd
        save_file({k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}, dst, {"format": "pt"})
    else:
        raise click.UsageError("unsupported conversion")
    click.echo(f"wrote {dst}")


@cli.command("models")
@click.option("--dir", "cache_dir", default=None)
@click.option("--catalog", "show_catalog", is_flag=True, help="list the built-in catalog instead of what is on disk")
def list_models(cache_dir, show_catalog):
    """List checkpoints in the model cache directory (or the catalog of known models)."""
    from ..assets.catalog import ModelCacheStore, ModelCatalog
    if show_catalog:
        for e in ModelCatalog().entries():
            click.echo(f"{e.id:32s} {e.modality.value:11s} {e.family:10s} {e.repo}")
        return
    store = ModelCacheStore(cache_dir or config.get("model_cache_dir"))
    rows = store.list()
    if not rows:
        click.echo(f"(nothing in {store.root})")
    for r in rows:
        click.echo(f"{r['id']:40s} {r['bytes'] / 2 ** 30:8.2f} GiB  {r.get('source', '')}")


@cli.command()
@click.argument("name")
@click.option("--from", "src", default=None, help="register a checkpoint that is already on disk instead of downloading")
@click.option("--copy", is_flag=True, help="copy instead of linking (with --from)")
@click.option("--dir", "cache_dir", default=None)
@click.option("--token", default=None, envvar="HF_TOKEN")
def pull(name, src, copy, cache_dir, token):
    """Fetch a catalog model or a Hugging Face repository into the model cache."""
    from ..assets.catalog import ModelCacheStore, ModelResolver
    store = ModelCacheStore(cache_dir or config.get("model_cache_dir"))
    res = ModelResolver(store=store)
    if src:
        entry = res.catalog.find(name)
        click.echo(str(store.add_local(entry.id if entry else name, src, link=not copy)))
        return
    click.echo(str(res.pull(name, token)))


cli.add_command(list_models, "list")


@cli.command()
def flags():
    """Print every runtime flag (environment variable, type, default, description)."""
    click.echo(config.describe())


@cli.command()
@click.option("--kind", default="llm", type=click.Choice(["llm", "moe_llm", "image_dit", "video_dit"]))
@click.option("--weight-gb", default=70.0)
@click.option("--heads", default=64)
@click.option("--ffn", default=28672)
@click.option("--experts", default=0)
@click.option("--tokens", default=0)
@click.option("--true-cfg", is_flag=True)
@click.option("--gpus", default=8)
def plan(kind, weight_gb, heads, ffn, experts, tokens, true_cfg, gpus):
    """Suggest a parallel layout for a model shape on N GPUs."""
    from ..engine import planner as P
    p = P.suggest(P.ModelShape(kind, int(weight_gb * 1e9), heads, heads, ffn, 0, experts, tokens, true_cfg), gpus)
    click.echo(p.describe())
