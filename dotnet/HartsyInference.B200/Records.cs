// Request / result records with the reference's names and defaults
// (HartsyInference.Engine: Requests/, Dispatch/ModelSpec.cs, Dispatch/Modality.cs, EngineOptions.cs).
using System;
using System.Collections.Generic;

namespace HartsyInference;

public class HartsyInferenceException : Exception { public HartsyInferenceException(string m) : base(m) { } }
public sealed class OutOfVramException : HartsyInferenceException { public OutOfVramException(string m) : base(m) { } }
public sealed class UnsupportedModelException : HartsyInferenceException { public UnsupportedModelException(string m) : base(m) { } }

public enum Modality { Text, Image, Video, Music, Speech, Transcribe, VoiceConversion, Fx, Vision, Restore, Mesh, World, Embeddings }
public enum StopReason { Stop, Length, ToolCall, Cancelled, Error }
public enum TextChunkKind { Chunk, Result, Status, StopReason, NativeToolCall }

public sealed record ModelSpec(string Requested, Modality Modality = Modality.Text, string? Catalog = null,
                               string? LocalPath = null, Dictionary<string, string>? Aux = null);

public sealed record EngineOptions
{
    public string ModelCacheDirectory { get; init; } = "~/.hartsyinference/models";
    public bool LowVram { get; init; }
    /// <summary>Parallel layout, e.g. "tp8", "sp4+cfg2", "single".</summary>
    public string Placement { get; init; } = "single";
    public int KvPageSize { get; init; } = 16;
    public long KvPoolBytesBudget { get; init; }
    public int MaxBatch { get; init; } = 256;
    public int MaxModelLen { get; init; } = 8192;
}

public sealed record ChatMessage(string role, string content);

public sealed record TextRequest
{
    public List<ChatMessage> Messages { get; init; } = new();
    public string? Prompt { get; init; }
    public float Temperature { get; init; } = 0.7f;
    public float TopP { get; init; } = 0.95f;
    public int TopK { get; init; }
    public float MinP { get; init; }
    public float RepetitionPenalty { get; init; } = 1.0f;
    public int MaxTokens { get; init; } = 4096;
    public int? Seed { get; init; }
    public bool Greedy { get; init; }
    public bool? EnableThinking { get; init; }
    public bool GraphDecode { get; init; } = true;
    public bool SpeculativeDecode { get; init; }
    public List<string> Stop { get; init; } = new();
    public bool JsonMode { get; init; }
}

public sealed record TextResult(string Text, IReadOnlyList<int> TokenIds, int PromptTokens, int CompletionTokens,
                                StopReason StopReason, double TtftSeconds, double TotalSeconds, string? Error);

public sealed record TextChunk(TextChunkKind Kind, string Text = "", TextResult? Result = null, StopReason? StopReason = null);

public sealed record ImageRequest
{
    public string Prompt { get; init; } = "";
    public string NegativePrompt { get; init; } = "";
    public int Width { get; init; } = 1024;
    public int Height { get; init; } = 1024;
    public int Steps { get; init; } = 20;
    public float Guidance { get; init; } = 3.5f;
    public float CfgScale { get; init; } = 1.0f;
    public long? Seed { get; init; }
}

public sealed record StepPreview(int Step, int TotalSteps);
public sealed record ImageResult(byte[] Rgb, int Width, int Height, long Seed, Dictionary<string, object>? Meta = null);

public sealed record VideoRequest
{
    public string Prompt { get; init; } = "";
    public string NegativePrompt { get; init; } = "";
    public int Width { get; init; } = 832;
    public int Height { get; init; } = 480;
    public int Frames { get; init; } = 81;
    public int Fps { get; init; } = 16;
    public int Steps { get; init; } = 50;
    public float CfgScale { get; init; } = 5.0f;
    public long? Seed { get; init; }
}

public sealed record VideoGenerationResult(IReadOnlyList<byte[]> Frames, int Width, int Height, byte[]? Audio, int Fps, long Seed);

public sealed record AudioRequest
{
    public string? Language { get; init; }
    public string Task { get; init; } = "transcribe";
    public bool Timestamps { get; init; } = true;
}

public sealed record TranscriptSegment(double Start, double End, string Text);

public sealed record TranscriptResult(string Text, string? Language, double Duration, IReadOnlyList<TranscriptSegment> Segments);

public sealed record MusicRequest
{
    public string Prompt { get; init; } = "";
    public float Seconds { get; init; } = 5f;
    public float Guidance { get; init; } = 3f;
    public bool Greedy { get; init; }
    public int Seed { get; init; }
}

public sealed record SpeechRequest
{
    public string Text { get; init; } = "";
    public string? Voice { get; init; }
    public float? Speed { get; init; }
}

public sealed record AudioResult(float[] Samples, int SampleRate);

public sealed record RestoreRequest
{
    public string Operation { get; init; } = "upscale";
    public int Tile { get; init; } = 128;
    public float TileOverlap { get; init; } = 0.25f;
}

public static class Records
{
    /// <summary>The native side answers in snake_case JSON.</summary>
    public static readonly System.Text.Json.JsonSerializerOptions SnakeCase = new()
    {
        PropertyNamingPolicy = System.Text.Json.JsonNamingPolicy.SnakeCaseLower,
        PropertyNameCaseInsensitive = true,
    };
}
