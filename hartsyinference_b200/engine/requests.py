"""Public request / result records of the engine.

Field names and defaults follow the reference's records so that the C ABI and the .NET facade can
stay source-compatible with it: ``TextRequest`` (Messages, Temperature 0.7, TopP 0.95, TopK, MinP,
RepetitionPenalty, MaxTokens 4096, Seed, Greedy, EnableThinking, Device, Tools, GraphDecode,
SpeculativeDecode), ``TextResult``, ``TextChunk{Kind}``, ``StopReason``, ``ImageRequest`` /
``ImageResult{Rgb, Width, Height, Seed, Meta}``, ``VideoRequest`` / ``VideoGenerationResult{Frames,
Audio, Fps}``, ``StepPreview``, ``ModelSpec{Requested, Modality, Catalog, LocalPath, Aux}``,
``EngineOptions{ModelCacheDirectory, LowVram, Placement, KvPageSize 16, KvPoolBytesBudget}``
(src/HartsyInference.Engine/Requests/, Dispatch/ModelSpec.cs, Dispatch/Modality.cs, EngineOptions.cs).
"""
from __future__ import annotations

import enum
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

from ..parallel.config import ParallelConfig


class Modality(str, enum.Enum):
    TEXT = "text"
    IMAGE = "image"
    VIDEO = "video"
    MUSIC = "music"
    SPEECH = "speech"
    TRANSCRIBE = "transcribe"
    VOICE_CONVERSION = "voice_conversion"
    FX = "fx"
    VISION = "vision"
    RESTORE = "restore"
    MESH = "mesh"
    WORLD = "world"
    EMBEDDINGS = "embeddings"


class StopReason(str, enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    TOOL_CALL = "tool_call"
    CANCELLED = "cancelled"
    ERROR = "error"


class ChunkKind(str, enum.Enum):
    CHUNK = "chunk"
    RESULT = "result"
    STATUS = "status"
    STOP_REASON = "stop_reason"
    NATIVE_TOOL_CALL = "native_tool_call"


@dataclass
class ModelSpec:
    requested: str                       # what the caller asked for (name, alias or path)
    modality: Modality = Modality.TEXT
    catalog: Optional[str] = None        # catalog id when resolved from the registry
    local_path: Optional[str] = None     # resolved checkpoint path
    aux: dict[str, str] = field(default_factory=dict)   # side models: vae, text_encoder, mmproj, ...


@dataclass
class EngineOptions:
    model_cache_directory: str = "~/.hartsyinference/models"
    low_vram: bool = False
    placement: ParallelConfig = field(default_factory=ParallelConfig)
    kv_page_size: int = 16
    kv_pool_bytes_budget: int = 0        # 0 = size the pool from free device memory
    max_batch: int = 256
    max_model_len: int = 8192


@dataclass
class TextRequest:
    messages: list[dict] = field(default_factory=list)
    prompt: Optional[str] = None         # raw prompt (bypasses the chat template)
    prompt_token_ids: Optional[list[int]] = None   # already tokenised prompt (bypasses template and tokenizer)
    ignore_eos: bool = False             # keep generating up to max_tokens (throughput measurements)
    temperature: float = 0.7
    top_p: float = 0.95
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 4096
    seed: Optional[int] = None
    greedy: bool = False
    enable_thinking: Optional[bool] = None
    device: Optional[str] = None
    tools: Optional[list] = None
    force_tool_id: Optional[str] = None
    graph_decode: bool = True
    speculative_decode: bool = False
    stop: list[str] = field(default_factory=list)
    json_mode: bool = False
    images: list = field(default_factory=list)   # one per "<image>" in the prompt (path, PIL image, array or tensor)


@dataclass
class TextResult:
    text: str = ""
    token_ids: list[int] = field(default_factory=list)
    prompt_tokens: int = 0
    completion_tokens: int = 0
    stop_reason: StopReason = StopReason.STOP
    ttft_s: float = 0.0
    total_s: float = 0.0
    error: Optional[str] = None
    tool_calls: list = field(default_factory=list)     # assets.tool_calls.ToolCall, when tools were offered

    @property
    def tokens_per_second(self) -> float:
        dt = self.total_s - self.ttft_s
        return (self.completion_tokens - 1) / dt if dt > 0 and self.completion_tokens > 1 else 0.0


@dataclass
class TextChunk:
    kind: ChunkKind
    text: str = ""
    result: Optional[TextResult] = None
    stop_reason: Optional[StopReason] = None
    status: Optional[str] = None


@dataclass
class ImageRequest:
    prompt: str = ""
    negative_prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int = 20
    guidance: float = 3.5
    cfg_scale: float = 1.0               # > 1 runs true classifier-free guidance (two branches)
    seed: Optional[int] = None
    sampler: str = "euler"
    scheduler: str = "flow_match_euler"
    batch: int = 1
    init_image: Optional[Any] = None
    mask_image: Optional[Any] = None     # white = repaint (inpainting; needs init_image)
    control_image: Optional[Any] = None  # ControlNet conditioning image (needs a ControlNet beside the model)
    image_prompt: Optional[Any] = None   # picture prompt (IP-Adapter on U-Net models, Redux on Flux)
    image_prompt_scale: float = 1.0
    control_strength: float = 1.0
    strength: float = 1.0
    loras: list[tuple[str, float]] = field(default_factory=list)
    step_cache_threshold: float = 0.0
    guidance_interval: Optional[tuple] = None   # (start, end) in [0, 1]: true CFG only on those steps (None: all)
    cfg_renorm_min: Optional[float] = None      # true CFG: rescale the guided prediction by clamp(|cond| / |guided|, this, 1)
    cfg_row_norm: bool = False                  # true CFG: rescale every guided row to the norm of its conditional row
    preview_every: int = 0               # > 0: every n-th step callback carries a small RGB preview of the latents
    vae_tile: int = 0                    # > 0: decode in latent tiles of this size (bounded activation memory)


@dataclass
class AudioRequest:
    """Speech-to-text input: a WAV path / bytes, or samples with their rate."""
    audio: Optional[Any] = None          # path, bytes, or float tensor [n] / [channels, n]
    sample_rate: int = 16000
    language: Optional[str] = None
    task: str = "transcribe"             # or "translate"
    timestamps: bool = True


@dataclass
class SpeechRequest:
    """Text-to-speech input. ``speed`` > 1 talks faster; the noise scales default to the voice's own."""
    text: str = ""
    voice: Optional[str] = None
    speed: Optional[float] = None
    noise_scale: Optional[float] = None
    noise_scale_duration: Optional[float] = None
    seed: int = 0                      # sampling models (Bark, CSM)
    greedy: bool = False
    max_seconds: float = 30.0          # autoregressive models stop here if no end frame came


@dataclass
class MusicRequest:
    """Text-to-music input (MusicGen). ``guidance`` is the classifier-free guidance scale; sampling
    draws from the top-k tokens, greedy decoding is deterministic."""
    prompt: str = ""
    seconds: float = 5.0
    guidance: float = 3.0
    greedy: bool = False
    seed: int = 0


@dataclass
class RestoreRequest:
    """``operation``: "upscale" (Real-ESRGAN). ``image``: path, PIL image, uint8 HWC array or float CHW tensor."""
    operation: str = "upscale"
    image: Optional[Any] = None
    tile: int = 128                      # input-space tile size; 0 = whole image at once
    tile_overlap: float = 0.25


@dataclass
class MeshRequest:
    """Single image -> mesh. ``image``: path, PIL image, uint8 HWC array or float CHW tensor (RGBA inputs
    are composited on mid-grey). ``resolution``: lattice points per axis (0 = the model's default);
    ``threshold``: density iso level (None = the model's default)."""
    image: Optional[Any] = None
    resolution: int = 0
    threshold: Optional[float] = None
    foreground_ratio: float = 0.85
    output_path: Optional[str] = None    # .obj / .ply / .glb


@dataclass
class MeshResult:
    vertices: Any = None                 # float32 [V, 3]
    faces: Any = None                    # int64 [F, 3]
    colors: Any = None                   # float32 [V, 3] in [0, 1]
    meta: dict = field(default_factory=dict)

    def save(self, path: str) -> None:
        from ..threed import writers
        ext = str(path).lower().rsplit(".", 1)[-1]
        if ext == "obj":
            writers.write_obj(path, self.vertices, self.faces)
        elif ext == "ply":
            writers.write_ply(path, self.vertices, self.faces, self.colors)
        elif ext == "glb":
            writers.write_glb(path, self.vertices, self.faces, colors=self.colors)
        else:
            raise ValueError(f"unknown mesh format '.{ext}' (obj, ply, glb)")


@dataclass
class WorldRequest:
    """First picture + one action row per frame to generate. ``image``: path, PIL image, uint8 HWC array
    or float CHW tensor; ``actions``: rows of 25 floats (Oasis: 23 keys / buttons, then the two camera
    deltas)."""
    image: Optional[Any] = None
    actions: list = field(default_factory=list)
    seed: Optional[int] = None


@dataclass
class WorldResult:
    frames: Any = None                   # float32 [N, 3, H, W] in [0, 1], the first picture's reconstruction included
    meta: dict = field(default_factory=dict)


@dataclass
class VisionRequest:
    """``operation``: "embed" (CLIP / SigLIP / DINOv2 image features, CLIP text features and their
    similarity when both are given), "depth" (Depth Anything; one map per image) or "segment" (CLIPSeg:
    one probability map per (image, text) pair) or "detect" (OWL-ViT: boxes for each text query above
    ``score_threshold``, after per-query non-maximum suppression)."""
    operation: str = "embed"
    images: list = field(default_factory=list)
    texts: list[str] = field(default_factory=list)
    score_threshold: float = 0.1
    nms_iou: float = 0.5
    # promptable segmentation (SAM 2): one mask per prompt; a prompt is a list of [x, y] points with their
    # labels (1 foreground, 0 background), a box [x0, y0, x1, y1], or both, in pixels of the image
    points: list = field(default_factory=list)        # per prompt: [[x, y], ...]
    point_labels: list = field(default_factory=list)  # per prompt: [1, 0, ...] (default: all foreground)
    boxes: list = field(default_factory=list)         # per prompt: [x0, y0, x1, y1]
    # "annotate": control pictures for ControlNets. ``annotator``: "canny" / "tile" / "blur" (no model needed),
    # "pose" (a pose checkpoint), "depth" (a depth checkpoint), "segmentation" (a scene-parsing checkpoint)
    annotator: str = "canny"
    canny_low: float = 100.0
    canny_high: float = 200.0


@dataclass
class VisionResult:
    image_embeddings: Optional[Any] = None     # [n_images, dim], L2-normalised
    text_embeddings: Optional[Any] = None      # [n_texts, dim]
    similarity: Optional[Any] = None           # [n_images, n_texts] cosine
    depth: Optional[list] = None               # per image: float32 [H, W] at the image's own size
    masks: Optional[list] = None               # per image: float32 [n_texts, H, W] probabilities in [0, 1]
    detections: Optional[list] = None          # per image: [{"label", "score", "box": [x0, y0, x1, y1] in pixels}]
    mask_scores: Optional[list] = None         # promptable segmentation, per image: predicted IoU of every returned mask
    labels: Optional[list] = None              # scene parsing, per image: names of the classes present (masks hold int64 label maps)
    control_images: Optional[list] = None      # annotate, per image: uint8 [H, W, 3]


@dataclass
class StepPreview:
    step: int
    total_steps: int
    latents: Optional[Any] = None
    preview_rgb: Optional[bytes] = None  # RGB24 at latent resolution (preview_width x preview_height)
    preview_width: int = 0
    preview_height: int = 0


@dataclass
class ImageResult:
    rgb: bytes = b""                     # RGB24, row-major
    width: int = 0
    height: int = 0
    seed: int = 0
    meta: dict = field(default_factory=dict)


@dataclass
class VideoRequest:
    prompt: str = ""
    negative_prompt: str = ""
    width: int = 832
    height: int = 480
    frames: int = 81
    fps: int = 16
    steps: int = 50
    cfg_scale: float = 5.0
    seed: Optional[int] = None
    scheduler: str = "unipc"
    shift: float = 5.0


@dataclass
class VideoGenerationResult:
    frames: list = field(default_factory=list)      # list of RGB24 byte strings
    width: int = 0
    height: int = 0
    audio: Optional[bytes] = None
    fps: int = 16
    seed: int = 0
    meta: dict = field(default_factory=dict)


def to_jsonable(obj) -> Any:
    if isinstance(obj, enum.Enum):
        return obj.value
    if hasattr(obj, "__dataclass_fields__"):
        return {k: to_jsonable(v) for k, v in asdict(obj).items()}
    if isinstance(obj, (list, tuple)):
        return [to_jsonable(v) for v in obj]
    if isinstance(obj, dict):
        return {k: to_jsonable(v) for k, v in obj.items()}
    if isinstance(obj, bytes):
        return None
    return obj
