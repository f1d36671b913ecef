// InferenceEngine facade with the reference's shape: new InferenceEngine(selector, options),
// service properties (Text, Images, Video, Embeddings), SetBackend, FreeMemory, IsSupported.
// (Reference: src/HartsyInference.Engine/InferenceEngine.cs, Services/IInferenceEngine.cs:6-45.)
using System;
using System.Collections.Generic;
using System.Runtime.CompilerServices;
using System.Runtime.InteropServices;
using System.Text.Json;
using System.Threading;
using System.Threading.Channels;
using System.Threading.Tasks;
using HartsyInference.Native;

namespace HartsyInference;

public interface IInferenceEngine : IDisposable
{
    string BackendSelector { get; }
    string BackendDescription { get; }
    TextService Text { get; }
    ImagesService Images { get; }
    VideoService Video { get; }
    TranscribeService Transcribe { get; }
    SpeechService Speech { get; }
    MusicService Music { get; }
    EmbeddingService Embeddings { get; }
    VisionService Vision { get; }
    RestoreService Restore { get; }
    void SetBackend(string selector);
    void FreeMemory();
    bool IsSupported(Modality modality);
}

public sealed class InferenceEngine : IInferenceEngine
{
    internal IntPtr Handle;
    public string BackendSelector { get; private set; }
    public TextService Text { get; }
    public ImagesService Images { get; }
    public VideoService Video { get; }
    public TranscribeService Transcribe { get; }
    public SpeechService Speech { get; }
    public MusicService Music { get; }
    public EmbeddingService Embeddings { get; }
    public VisionService Vision { get; }
    public RestoreService Restore { get; }

    public InferenceEngine(string backendSelector = "auto", EngineOptions? options = null)
    {
        BackendSelector = backendSelector;
        NativeMethods.Check(NativeMethods.b200_engine_create(backendSelector, JsonSerializer.Serialize(options ?? new EngineOptions()), out Handle));
        Text = new TextService(this);
        Images = new ImagesService(this);
        Video = new VideoService(this);
        Transcribe = new TranscribeService(this);
        Speech = new SpeechService(this);
        Music = new MusicService(this);
        Embeddings = new EmbeddingService(this);
        Vision = new VisionService(this);
        Restore = new RestoreService(this);
    }

    public string BackendDescription
    {
        get
        {
            NativeMethods.Check(NativeMethods.b200_engine_describe(Handle, out var p));
            using var doc = JsonDocument.Parse(NativeMethods.TakeString(p));
            return doc.RootElement.GetProperty("backend_description").GetString() ?? "";
        }
    }

    public void SetBackend(string selector)
    {
        NativeMethods.Check(NativeMethods.b200_engine_set_backend(Handle, selector));
        BackendSelector = selector;
    }

    public void FreeMemory() => NativeMethods.Check(NativeMethods.b200_free_memory(Handle));

    public bool IsSupported(Modality modality) => NativeMethods.b200_engine_is_supported(Handle, modality.ToString().ToLowerInvariant()) != 0;

    public void Dispose()
    {
        if (Handle != IntPtr.Zero) { NativeMethods.b200_engine_destroy(Handle); Handle = IntPtr.Zero; }
    }
}

public sealed class TextService
{
    private readonly InferenceEngine _e;
    internal TextService(InferenceEngine e) => _e = e;

    public Task<TextResult> GenerateAsync(ModelSpec spec, TextRequest request, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_text_generate(_e.Handle, JsonSerializer.Serialize(spec), JsonSerializer.Serialize(request), out var p));
        return ParseResult(NativeMethods.TakeString(p));
    }, ct);

    public async IAsyncEnumerable<TextChunk> StreamAsync(ModelSpec spec, TextRequest request, [EnumeratorCancellation] CancellationToken ct = default)
    {
        var channel = Channel.CreateUnbounded<TextChunk>();
        NativeMethods.ChunkCallback cb = (kind, payload, _) =>
        {
            string k = Marshal.PtrToStringUTF8(kind) ?? "", v = Marshal.PtrToStringUTF8(payload) ?? "";
            channel.Writer.TryWrite(k switch
            {
                "chunk" => new TextChunk(TextChunkKind.Chunk, v),
                "result" => new TextChunk(TextChunkKind.Result, Result: ParseResult(v)),
                "stop_reason" => new TextChunk(TextChunkKind.StopReason, StopReason: ParseStop(v)),
                _ => new TextChunk(TextChunkKind.Status, v),
            });
            return ct.IsCancellationRequested ? 1 : 0;
        };
        var worker = Task.Run(() =>
        {
            try { NativeMethods.Check(NativeMethods.b200_text_stream(_e.Handle, JsonSerializer.Serialize(spec), JsonSerializer.Serialize(request), cb, IntPtr.Zero)); }
            finally { channel.Writer.TryComplete(); GC.KeepAlive(cb); }
        });
        await foreach (var chunk in channel.Reader.ReadAllAsync(ct)) yield return chunk;
        await worker;
    }

    public int CountTokens(ModelSpec spec, TextRequest request)
    {
        NativeMethods.Check(NativeMethods.b200_text_count_tokens(_e.Handle, JsonSerializer.Serialize(spec), JsonSerializer.Serialize(request), out int n));
        return n;
    }

    private static StopReason ParseStop(string s) => s switch
    {
        "length" => StopReason.Length, "tool_call" => StopReason.ToolCall, "cancelled" => StopReason.Cancelled,
        "error" => StopReason.Error, _ => StopReason.Stop,
    };

    private static TextResult ParseResult(string json)
    {
        using var doc = JsonDocument.Parse(json);
        var r = doc.RootElement;
        var ids = new List<int>();
        foreach (var t in r.GetProperty("token_ids").EnumerateArray()) ids.Add(t.GetInt32());
        return new TextResult(r.GetProperty("text").GetString() ?? "", ids, r.GetProperty("prompt_tokens").GetInt32(),
            r.GetProperty("completion_tokens").GetInt32(), ParseStop(r.GetProperty("stop_reason").GetString() ?? "stop"),
            r.GetProperty("ttft_s").GetDouble(), r.GetProperty("total_s").GetDouble(),
            r.TryGetProperty("error", out var e) && e.ValueKind == JsonValueKind.String ? e.GetString() : null);
    }
}

public sealed class ImagesService
{
    private readonly InferenceEngine _e;
    internal ImagesService(InferenceEngine e) => _e = e;

    public Task<ImageResult> GenerateAsync(ModelSpec spec, ImageRequest request, IProgress<StepPreview>? progress = null, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.StepCallback cb = (step, total, _) => { progress?.Report(new StepPreview(step, total)); return ct.IsCancellationRequested ? 1 : 0; };
        NativeMethods.Check(NativeMethods.b200_image_generate(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Image }),
            JsonSerializer.Serialize(request), cb, IntPtr.Zero, out var rgb, out int w, out int h, out long seed));
        try
        {
            var bytes = new byte[w * h * 3];
            Marshal.Copy(rgb, bytes, 0, bytes.Length);
            return new ImageResult(bytes, w, h, seed);
        }
        finally { NativeMethods.b200_free(rgb); GC.KeepAlive(cb); }
    }, ct);
}

public sealed class VideoService
{
    private readonly InferenceEngine _e;
    internal VideoService(InferenceEngine e) => _e = e;

    public Task<VideoGenerationResult> GenerateAsync(ModelSpec spec, VideoRequest request, IProgress<StepPreview>? progress = null, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.StepCallback cb = (step, total, _) => { progress?.Report(new StepPreview(step, total)); return ct.IsCancellationRequested ? 1 : 0; };
        NativeMethods.Check(NativeMethods.b200_video_generate(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Video }),
            JsonSerializer.Serialize(request), cb, IntPtr.Zero, out var buf, out int n, out int w, out int h, out int fps, out long seed));
        try
        {
            var frames = new List<byte[]>(n);
            int size = w * h * 3;
            for (int i = 0; i < n; i++) { var f = new byte[size]; Marshal.Copy(buf + i * size, f, 0, size); frames.Add(f); }
            return new VideoGenerationResult(frames, w, h, null, fps, seed);
        }
        finally { NativeMethods.b200_free(buf); GC.KeepAlive(cb); }
    }, ct);
}

public sealed class TranscribeService
{
    private readonly InferenceEngine _e;
    internal TranscribeService(InferenceEngine e) => _e = e;

    /// <summary>Mono float samples in [-1, 1] at <paramref name="sampleRate"/> Hz -> transcript JSON mapped onto <see cref="TranscriptResult"/>.</summary>
    public Task<TranscriptResult> RunAsync(ModelSpec spec, AudioRequest request, float[] pcm, int sampleRate, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_transcribe(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Transcribe }),
            JsonSerializer.Serialize(request), pcm, pcm.LongLength, sampleRate, out var p));
        return JsonSerializer.Deserialize<TranscriptResult>(NativeMethods.TakeString(p), Records.SnakeCase)!;
    }, ct);
}

public sealed class MusicService
{
    private readonly InferenceEngine _e;
    internal MusicService(InferenceEngine e) => _e = e;

    public Task<AudioResult> RunAsync(ModelSpec spec, MusicRequest request, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_music(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Music }),
            JsonSerializer.Serialize(request), out var pcm, out long n, out int rate));
        try
        {
            var samples = new float[n];
            Marshal.Copy(pcm, samples, 0, (int)n);
            return new AudioResult(samples, rate);
        }
        finally { NativeMethods.b200_free(pcm); }
    }, ct);
}

public sealed class SpeechService
{
    private readonly InferenceEngine _e;
    internal SpeechService(InferenceEngine e) => _e = e;

    public Task<AudioResult> RunAsync(ModelSpec spec, SpeechRequest request, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_speak(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Speech }),
            JsonSerializer.Serialize(request), out var pcm, out long n, out int rate));
        try
        {
            var samples = new float[n];
            Marshal.Copy(pcm, samples, 0, (int)n);
            return new AudioResult(samples, rate);
        }
        finally { NativeMethods.b200_free(pcm); }
    }, ct);
}

public sealed class EmbeddingService
{
    private readonly InferenceEngine _e;
    internal EmbeddingService(InferenceEngine e) => _e = e;

    public Task<float[][]> EmbedAsync(ModelSpec spec, IReadOnlyList<string> texts, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_embed_text(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Embeddings }),
            JsonSerializer.Serialize(texts), out var buf, out int count, out int dim));
        try
        {
            var rows = new float[count][];
            for (int i = 0; i < count; i++) { rows[i] = new float[dim]; Marshal.Copy(buf + i * dim * sizeof(float), rows[i], 0, dim); }
            return rows;
        }
        finally { NativeMethods.b200_free(buf); }
    }, ct);
}

public sealed class VisionService
{
    private readonly InferenceEngine _e;
    internal VisionService(InferenceEngine e) => _e = e;

    /// <summary>L2-normalised embedding of one RGB24 image (CLIP / SigLIP / DINOv2 checkpoints).</summary>
    public Task<float[]> EmbedImageAsync(ModelSpec spec, byte[] rgb, int width, int height, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_embed_image(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Vision }),
            rgb, width, height, out var buf, out int dim));
        try { var v = new float[dim]; Marshal.Copy(buf, v, 0, dim); return v; }
        finally { NativeMethods.b200_free(buf); }
    }, ct);
}

public sealed class RestoreService
{
    private readonly InferenceEngine _e;
    internal RestoreService(InferenceEngine e) => _e = e;

    public Task<ImageResult> UpscaleAsync(ModelSpec spec, RestoreRequest request, byte[] rgb, int width, int height, CancellationToken ct = default) => Task.Run(() =>
    {
        NativeMethods.Check(NativeMethods.b200_upscale(_e.Handle, JsonSerializer.Serialize(spec with { Modality = Modality.Restore }),
            JsonSerializer.Serialize(request), rgb, width, height, out var outBuf, out int w, out int h));
        try { var bytes = new byte[w * h * 3]; Marshal.Copy(outBuf, bytes, 0, bytes.Length); return new ImageResult(bytes, w, h, 0); }
        finally { NativeMethods.b200_free(outBuf); }
    }, ct);
}
