// Drop-in replacement of NFAI.Models.Llama3/LlamaModel.cs over libnfai_cuda.so. Public surface as in the reference
// (lines 10-175): ModelName, Dispose, GetStreamingResponseAsync, RunAsync. What changes is inside:
//  * the constructor (reference :21-68) reads the same metadata keys, then hands geometry and tensors to a
//    CudaLlamaBackend instead of building a TokenEmbed shader, N TransformerBlocks, an RMSNorm and a tied LM head;
//  * the prompt loop (reference :103-126) is one Prefill call, each decode iteration (:134-173) one Decode call;
//  * sampling runs on the device over the step's logits with a host-drawn uniform number (same algorithm and
//    defaults as SamplingUtils.TopP, SamplingUtils.cs:5-33); set NFAI_HOST_SAMPLING=1 to read the logits back and
//    call SamplingUtils.TopP exactly as the reference does, or NFAI_GREEDY=1 for SamplingUtils.ArgMax semantics;
//  * Dispose releases the device memory (the reference throws NotImplementedException, :70-74);
//  * a prompt that does not fit the KV cache raises InvalidOperationException (the reference writes out of bounds).
using System.Runtime.CompilerServices;
using Microsoft.Extensions.AI;
using NFAI.Core;
using NFAI.Cuda;

namespace NFAI.Models.Llama3;

public class LlamaModel : IInferenceProvider
{
    private readonly Tokenizer tokenizer;
    private readonly CudaLlamaBackend backend;
    private readonly bool hostSampling = Environment.GetEnvironmentVariable("NFAI_HOST_SAMPLING") == "1";
    private readonly bool greedy = Environment.GetEnvironmentVariable("NFAI_GREEDY") == "1";
    private bool firstInput = true;

    public string ModelName { get; init; }

    public LlamaModel(CudaContext cuda, Dictionary<string, object> metadata, List<AbstractComputeCollection> tensors, uint contextSize = 1024u)
    {
        // the keys the reference constructor reads (:23-34); bos/eos are consumed by the Tokenizer
        var ropeBase = (float)metadata["llama.rope.freq_base"];
        var ropeDim = (uint)metadata["llama.rope.dimension_count"];
        var eps = (float)(metadata.Where(kv => kv.Key.Contains("epsilon")).Select(kv => kv.Value).FirstOrDefault() ?? 0f);
        var qHeads = (uint)metadata["llama.attention.head_count"];
        var kvHeads = (uint)metadata["llama.attention.head_count_kv"];
        var headDim = (uint)metadata["llama.attention.key_length"];
        var layers = (uint)metadata["llama.block_count"];
        ModelName = metadata["general.name"].ToString() ?? "unknown";

        tokenizer = new Tokenizer(metadata);

        // the same look-ups by name fragment as the reference (:43,58 and TransformerBlock.cs:41-99)
        var embed = Find(tensors, "token") ?? throw new ArgumentException("token_embd.weight is missing");
        var gate0 = Find(tensors, "blk.0.ffn_gate") ?? throw new ArgumentException("blk.0.ffn_gate.weight is missing");
        var untiedHead = tensors.FirstOrDefault(t => t.Name == "output.weight");

        var hp = new NfaiHParams
        {
            H = (uint)embed.Shape[0], V = (uint)embed.Shape[1], L = layers, qH = qHeads, kvH = kvHeads, d = headDim,
            ropeDim = ropeDim, F = (uint)gate0.Shape[1], ctx = contextSize, eps = eps, rope_theta = ropeBase,
            weight_dtype = embed.TypeSize == 2 ? (int)NfaiDType.F16 : (int)NfaiDType.F32,  // float16 files stay float16 in HBM
            kv_dtype = KvCacheType(),
            tied = untiedHead == null ? 1 : 0,
        };
        backend = new CudaLlamaBackend(cuda, hp);

        Upload(embed);
        Upload(Find(tensors, "output_norm") ?? throw new ArgumentException("output_norm.weight is missing"));
        if (untiedHead != null) Upload(untiedHead);
        string[] perLayer = ["attn_norm", "attn_q", "attn_k", "attn_v", "attn_output.weight", "ffn_norm", "ffn_down", "ffn_gate", "ffn_up"];
        for (var i = 0u; i < layers; i++)
            foreach (var part in perLayer)
                Upload(Find(tensors, $"blk.{i}.{part}") ?? throw new ArgumentException($"blk.{i}.{part} is missing"));
        backend.FinalizeModel();
    }

    private static AbstractComputeCollection? Find(List<AbstractComputeCollection> tensors, string fragment) =>
        tensors.FirstOrDefault(t => t.Name.Contains(fragment));

    // FP32 like the reference's cache by default; NFAI_KV_F16=1 halves the cache traffic.
    private static int KvCacheType() =>
        Environment.GetEnvironmentVariable("NFAI_KV_F16") == "1" ? (int)NfaiDType.F16 : (int)NfaiDType.F32;

    // Parser.cs:101-110 hands every tensor over as ComputeCollection<float>; its GetDataRaw yields 10 MiB chunks with
    // halves already widened to float32 (AbstractComputeCollection.cs:36-79), which the library narrows back exactly.
    private void Upload(AbstractComputeCollection tensor)
    {
        var typed = tensor as ComputeCollection<float> ?? throw new ArgumentException($"{tensor.Name}: only F32/F16 tensors can be uploaded");
        backend.Upload(typed, typed.GetDataRaw(), chunksAreFloat32: true);
    }

    public void Dispose()
    {
        GC.SuppressFinalize(this);
        backend.Dispose();
    }

    public async IAsyncEnumerable<ChatResponseUpdate> GetStreamingResponseAsync(IEnumerable<ChatMessage> messages, ChatOptions? options = null, [EnumeratorCancellation] CancellationToken cancellationToken = default)
    {
        var user = messages.FirstOrDefault(m => m.Role == ChatRole.User) ?? throw new ArgumentException("No user message found in the input messages.");
        var messageId = Guid.NewGuid().ToString();
        await foreach (var piece in RunAsync(user.Text, cancellationToken))
            yield return new ChatResponseUpdate
            {
                CreatedAt = DateTime.UtcNow,
                ModelId = ModelName,
                MessageId = messageId,
                Contents = [new TextContent(piece)],
            };
    }

    private uint Pick(float[]? logits)
    {
        if (greedy) return logits != null ? SamplingUtils.ArgMax(logits) : backend.LastArgMax();
        return logits != null ? SamplingUtils.TopP(logits) : backend.SampleTopP();
    }

    public async IAsyncEnumerable<string> RunAsync(string prompt, [EnumeratorCancellation] CancellationToken ct = default)
    {
        var ids = tokenizer.Tokenize(prompt, addBos: firstInput);
        firstInput = false;
        // one batched pass over the prompt; its result equals the reference's token-by-token loop
        var logits = backend.Prefill(ids.ToArray(), wantLogits: hostSampling);
        var tk = Pick(logits);
        yield return tokenizer.Detokenize([tk]);
        while (tk != tokenizer.EosTokenId && !ct.IsCancellationRequested)
        {
            logits = backend.Decode(tk, wantLogits: hostSampling);
            tk = Pick(logits);
            if (tk != tokenizer.EosTokenId)
                yield return tokenizer.Detokenize([tk]);
            await Task.Yield();
        }
    }
}
