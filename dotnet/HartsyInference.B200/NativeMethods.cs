// P/Invoke table of libb200infer.so (see hartsyinference_b200/csrc/cabi/b200infer.h).
// This project has not been compiled in this repository's build environment: no .NET SDK is
// installed there. It is kept source-level in step with the header.
using System;
using System.Runtime.InteropServices;

namespace HartsyInference.Native;

internal static unsafe class NativeMethods
{
    private const string Lib = "b200infer";

    [UnmanagedFunctionPointer(CallingConvention.Cdecl)]
    internal delegate int ChunkCallback(IntPtr kind, IntPtr payload, IntPtr user);

    [UnmanagedFunctionPointer(CallingConvention.Cdecl)]
    internal delegate int StepCallback(int step, int total, IntPtr user);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_engine_create([MarshalAs(UnmanagedType.LPUTF8Str)] string selector,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string optionsJson, out IntPtr engine);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern void b200_engine_destroy(IntPtr engine);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_engine_set_backend(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string selector);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_engine_describe(IntPtr engine, out IntPtr json);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_engine_is_supported(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string modality);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_free_memory(IntPtr engine);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_text_generate(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, out IntPtr resultJson);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_text_stream(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, ChunkCallback cb, IntPtr user);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_text_count_tokens(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, out int tokens);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_image_generate(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, StepCallback? cb, IntPtr user,
        out IntPtr rgb, out int width, out int height, out long seed);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_video_generate(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, StepCallback? cb, IntPtr user,
        out IntPtr frames, out int frameCount, out int width, out int height, out int fps, out long seed);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_transcribe(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, float[] pcm, long samples, int sampleRate, out IntPtr resultJson);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_speak(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, out IntPtr pcm, out long samples, out int sampleRate);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_music(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, out IntPtr pcm, out long samples, out int sampleRate);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_embed_text(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string textsJson, out IntPtr values, out int count, out int dim);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_embed_image(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        byte[] rgb, int width, int height, out IntPtr values, out int dim);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern int b200_upscale(IntPtr engine, [MarshalAs(UnmanagedType.LPUTF8Str)] string spec,
        [MarshalAs(UnmanagedType.LPUTF8Str)] string request, byte[] rgb, int width, int height,
        out IntPtr rgbOut, out int widthOut, out int heightOut);

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern IntPtr b200_last_error();

    [DllImport(Lib, CallingConvention = CallingConvention.Cdecl)]
    internal static extern void b200_free(IntPtr p);

    internal static string TakeString(IntPtr p)
    {
        if (p == IntPtr.Zero) return string.Empty;
        try { return Marshal.PtrToStringUTF8(p) ?? string.Empty; }
        finally { b200_free(p); }
    }

    internal static void Check(int code)
    {
        if (code == 0) return;
        string msg = Marshal.PtrToStringUTF8(b200_last_error()) ?? "native error";
        throw code switch
        {
            2 => new OutOfVramException(msg),
            3 => new UnsupportedModelException(msg),
            _ => new HartsyInferenceException(msg),
        };
    }
}
