// The device side of LlamaModel: upload, prompt ingestion, decode. LlamaModel keeps its public shape
// (NFAI.Models.Llama3/LlamaModel.cs:10-175) and holds one of these instead of the shader objects.
using NFAI.Core;

namespace NFAI.Cuda;

public sealed unsafe class CudaLlamaBackend : IDisposable
{
    private readonly CudaContext ctx;
    private IntPtr model;
    public uint Vocab { get; }

    public CudaLlamaBackend(CudaContext ctx, NfaiHParams hp)
    {
        this.ctx = ctx;
        Vocab = hp.V;
        Native.Check(Native.nfai_model_create(ctx.Handle, in hp, out model), ctx.Handle);
    }

    // Streams one tensor exactly as the reference does for a shader property: the chunks GetDataRaw yields
    // (halves already widened to float32, NFAI.Core/AbstractComputeCollection.cs:36-79) go to the device.
    public void Upload(AbstractComputeCollection tensor, IEnumerable<byte[]> rawChunks, bool chunksAreFloat32)
    {
        var shape = tensor.Shape.Select(s => (ulong)s).ToArray();
        fixed (ulong* ps = shape)
            Native.Check(Native.nfai_model_tensor_begin(model, tensor.Name, chunksAreFloat32 ? 0 : 1, ps, shape.Length), ctx.Handle);
        foreach (var chunk in rawChunks)
            fixed (byte* pb = chunk)
                Native.Check(Native.nfai_model_tensor_chunk(model, pb, (nuint)chunk.Length), ctx.Handle);
        Native.Check(Native.nfai_model_tensor_end(model), ctx.Handle);
    }

    public void FinalizeModel() => Native.Check(Native.nfai_model_finalize(model), ctx.Handle);

    private uint lastArgMax;

    // Prompt loop of RunAsync (LlamaModel.cs:103-126) as one call. Returns the logits of the last prompt token, or
    // null when the caller does not want them read back (it then samples on the device or takes LastArgMax()).
    public float[]? Prefill(ReadOnlySpan<uint> tokens, bool wantLogits = true)
    {
        var logits = wantLogits ? new float[Vocab] : null;
        uint am;
        fixed (uint* pt = tokens) fixed (float* pl = logits)
            Native.Check(Native.nfai_prefill(model, pt, tokens.Length, pl, &am), ctx.Handle);
        lastArgMax = am;
        return logits;
    }

    // One iteration of the decode loop (LlamaModel.cs:134-173). With wantLogits the 4*V bytes go to
    // SamplingUtils.TopP on the host as in the reference; without, only the arg-max index crosses PCIe.
    public float[]? Decode(uint token, bool wantLogits = true)
    {
        var logits = wantLogits ? new float[Vocab] : null;
        uint am;
        fixed (float* pl = logits)
            Native.Check(Native.nfai_decode(model, token, pl, &am), ctx.Handle);
        lastArgMax = am;
        return logits;
    }

    // Index of the largest logit of the last Prefill/Decode, lowest index among equal maxima
    // (SamplingUtils.ArgMax, SamplingUtils.cs:43-57).
    public uint LastArgMax() => lastArgMax;

    public uint DecodeGreedy(uint token)
    {
        Decode(token, wantLogits: false);
        return lastArgMax;
    }

    // SamplingUtils.TopP (SamplingUtils.cs:5-33) on the device over the logits of the last Prefill/Decode: the 513 KB
    // logits read-back becomes a 4-byte token. The uniform draw stays on the host (Random.Shared, as today).
    public uint SampleTopP(float temperature = 0.5f, float topP = 0.95f, int topK = 40)
    {
        Native.Check(Native.nfai_sample_top_p(model, temperature, topP, topK, Random.Shared.NextSingle(), out uint tok), ctx.Handle);
        return tok;
    }

    // Multi-turn reuse: Prefill appends at the current position; a snapshot rewinds to an earlier point (for example
    // right after a shared system prompt) without ingesting it again.
    public IntPtr Snapshot()
    {
        Native.Check(Native.nfai_kv_snapshot_create(model, out IntPtr snap), ctx.Handle);
        return snap;
    }

    public void Restore(IntPtr snapshot) => Native.Check(Native.nfai_kv_snapshot_restore(model, snapshot), ctx.Handle);

    public static void FreeSnapshot(IntPtr snapshot) => Native.nfai_kv_snapshot_destroy(snapshot);

    public void Reset() => Native.Check(Native.nfai_reset(model), ctx.Handle);

    public void Dispose()
    {
        if (model != IntPtr.Zero) { Native.nfai_model_destroy(model); model = IntPtr.Zero; }
        GC.SuppressFinalize(this);
    }
}
