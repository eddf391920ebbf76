// P/Invoke declarations of include/nfai_cuda.h, one to one. Not compiled where this repository is developed
// (no .NET SDK there); the same call sequence is exercised through ctypes in nfai_b200/_lib.py.
using System.Runtime.InteropServices;

namespace NFAI.Cuda;

public enum NfaiStatus { Ok = 0, Arg = 1, State = 2, Oom = 3, Cuda = 4, Nccl = 5, ContextFull = 6, Timeout = 7 }
public enum NfaiDType { F32 = 0, F16 = 1 }

[StructLayout(LayoutKind.Sequential)]
public struct NfaiHParams
{
    public uint H, L, qH, kvH, d, ropeDim, F, V, ctx;
    public float eps, rope_theta;
    public int weight_dtype, kv_dtype, tied;
}

internal static unsafe partial class Native
{
    private const string Lib = "nfai_cuda"; // resolves to libnfai_cuda.so

    [DllImport(Lib)] internal static extern IntPtr nfai_version();
    [DllImport(Lib)] internal static extern IntPtr nfai_last_error(IntPtr ctx);
    [DllImport(Lib)] internal static extern int nfai_ctx_create(int deviceOrdinal, out IntPtr ctx);
    [DllImport(Lib)] internal static extern int nfai_tp_unique_id(byte* outId, nuint outBytes);
    [DllImport(Lib)] internal static extern int nfai_ctx_create_tp(int deviceOrdinal, int rank, int world, byte* uid, nuint uidBytes, out IntPtr ctx);
    [DllImport(Lib)] internal static extern int nfai_tp_export_peer(IntPtr ctx, byte* outDesc, nuint outBytes);
    [DllImport(Lib)] internal static extern int nfai_tp_import_peers(IntPtr ctx, byte* descs, int n);
    [DllImport(Lib)] internal static extern int nfai_ctx_destroy(IntPtr ctx);
    [DllImport(Lib)] internal static extern int nfai_ctx_set_wait_ns(IntPtr ctx, ulong ns);
    [DllImport(Lib)] internal static extern int nfai_model_create(IntPtr ctx, in NfaiHParams hp, out IntPtr model);
    [DllImport(Lib, CharSet = CharSet.Ansi)] internal static extern int nfai_model_tensor_begin(IntPtr model, string ggufName, int srcDType, ulong* shape, int ndim);
    [DllImport(Lib)] internal static extern int nfai_model_tensor_chunk(IntPtr model, byte* bytes, nuint nbytes);
    [DllImport(Lib)] internal static extern int nfai_model_tensor_end(IntPtr model);
    [DllImport(Lib)] internal static extern int nfai_model_finalize(IntPtr model);
    [DllImport(Lib, CharSet = CharSet.Ansi)] internal static extern int nfai_model_load_gguf(IntPtr ctx, string path, uint kvCacheSize, int kvDType, out IntPtr model);
    [DllImport(Lib, CharSet = CharSet.Ansi)] internal static extern int nfai_gguf_probe(string path, uint kvCacheSize, out NfaiHParams hp, byte* errOut, nuint errBytes);
    [DllImport(Lib)] internal static extern int nfai_model_get_hparams(IntPtr model, out NfaiHParams hp);
    [DllImport(Lib)] internal static extern int nfai_op_gemm_f16(IntPtr ctx, void* a, void* w, uint m, uint n, uint k, float* c);
    [DllImport(Lib)] internal static extern int nfai_model_destroy(IntPtr model);
    [DllImport(Lib)] internal static extern int nfai_prefill(IntPtr model, uint* tokens, int n, float* logitsLast, uint* argmaxLast);
    [DllImport(Lib)] internal static extern int nfai_decode(IntPtr model, uint token, float* logits, uint* argmax);
    [DllImport(Lib)] internal static extern int nfai_decode_greedy(IntPtr model, uint firstToken, int nSteps, uint* outTokens, float* elapsedMs);
    [DllImport(Lib)] internal static extern int nfai_sample_top_p(IntPtr model, float temperature, float topP, int topK, float u, out uint token);
    [DllImport(Lib)] internal static extern int nfai_op_sample_top_p(IntPtr ctx, IntPtr logits, uint V, float temperature, float topP, int topK, float u, IntPtr tokenOut);
    [DllImport(Lib)] internal static extern int nfai_decode_sampled(IntPtr model, uint firstToken, int nSteps, float temperature, float topP, int topK, float[] u, uint[] tokensOut, out float elapsedMs);
    [DllImport(Lib)] internal static extern int nfai_kv_snapshot_create(IntPtr model, out IntPtr snapshot);
    [DllImport(Lib)] internal static extern int nfai_kv_snapshot_restore(IntPtr model, IntPtr snapshot);
    [DllImport(Lib)] internal static extern void nfai_kv_snapshot_destroy(IntPtr snapshot);
    [DllImport(Lib)] internal static extern uint nfai_kv_snapshot_position(IntPtr snapshot);
    // host-side tokenizer (no GPU work): token / merge byte strings as arrays of pointers + lengths
    [DllImport(Lib)] internal static extern int nfai_tokenizer_create(IntPtr[] tokens, uint[] tokenLens, uint nTokens, IntPtr[] merges, uint[] mergeLens, uint nMerges, uint bosId, uint eosId, out IntPtr tokenizer);
    [DllImport(Lib)] internal static extern void nfai_tokenizer_destroy(IntPtr tokenizer);
    [DllImport(Lib)] internal static extern IntPtr nfai_tokenizer_last_error(IntPtr tokenizer);
    [DllImport(Lib)] internal static extern int nfai_tokenizer_encode(IntPtr tokenizer, byte[] textUtf8, nuint textLen, uint[] idsOut, nuint cap, out nuint n);
    [DllImport(Lib)] internal static extern int nfai_tokenizer_encode_chat(IntPtr tokenizer, byte[] promptUtf8, nuint promptLen, int addBos, uint[] idsOut, nuint cap, out nuint n);
    [DllImport(Lib)] internal static extern int nfai_tokenizer_pretokenize(IntPtr tokenizer, byte[] textUtf8, nuint textLen, uint[] endsOut, nuint cap, out nuint n);
    [DllImport(Lib)] internal static extern int nfai_tokenizer_decode(IntPtr tokenizer, uint[] ids, nuint n, byte[] textOut, nuint cap, out nuint nOut);
    [DllImport(Lib)] internal static extern int nfai_position(IntPtr model, out uint pos);
    [DllImport(Lib)] internal static extern int nfai_reset(IntPtr model);
    [DllImport(Lib)] internal static extern int nfai_set_position(IntPtr model, uint pos);
    [DllImport(Lib)] internal static extern int nfai_read_kv(IntPtr model, uint layer, uint pos, float* k, float* v);
    [DllImport(Lib)] internal static extern int nfai_write_kv(IntPtr model, uint layer, uint pos, float* k, float* v);
    [DllImport(Lib)] internal static extern int nfai_write_kv_range(IntPtr model, uint layer, uint pos0, uint n, float* k, float* v);
    [DllImport(Lib)] internal static extern int nfai_read_hidden(IntPtr model, uint layer, float* outHidden);
    [DllImport(Lib)] internal static extern int nfai_model_tune(IntPtr model, int which, int mode, int rowsPerWarp, int depth, int ctasPerSm);
    [DllImport(Lib)] internal static extern int nfai_model_set_prefetch(IntPtr model, ulong lookaheadBytes, ulong extraBytes, int mode);
    [DllImport(Lib)] internal static extern int nfai_op_attn_decode_static(IntPtr ctx, float* q, void* kcache, void* vcache, int kvDType, uint seq, uint qH, uint kvH, uint d, float* outp);
    [DllImport(Lib)] internal static extern int nfai_profile_kernel(IntPtr model, int which, int iters, out float avgMs, out ulong bytesPerLaunch);
    [DllImport(Lib)] internal static extern int nfai_step_launches(IntPtr model, out int launches);

    internal static void Check(int status, IntPtr ctx)
    {
        if (status == 0) return;
        string msg = Marshal.PtrToStringAnsi(nfai_last_error(ctx)) ?? string.Empty;
        throw new InvalidOperationException($"{(NfaiStatus)status}: {msg}");
    }
}
