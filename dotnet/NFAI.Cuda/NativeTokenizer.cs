// Drop-in for NFAI.Models.Llama3.Tokenizer (Tokenizer.cs) over the native byte-pair encoder of libnfai_cuda:
// same constructor input (the GGUF metadata), same Tokenize / Detokenize results and failures, without the scan over
// the whole merges list for every adjacent pair (Tokenizer.cs:130-166).
using System.Runtime.InteropServices;
using System.Text;

namespace NFAI.Cuda;

public sealed class NativeTokenizer : IDisposable
{
    private IntPtr handle;
    public uint BosTokenId { get; }
    public uint EosTokenId { get; }

    public NativeTokenizer(Dictionary<string, object> metadata)
    {
        var tokens = ((List<object>)metadata["tokenizer.ggml.tokens"])
            .Select(x => x switch { string s => Encoding.UTF8.GetBytes(s), byte[] b => b, _ => throw new Exception("Unexpected token format") })
            .ToList();
        var merges = ((List<object>)metadata["tokenizer.ggml.merges"]).Select(x => Encoding.UTF8.GetBytes((string)x)).ToList();
        BosTokenId = (uint)metadata["tokenizer.ggml.bos_token_id"];
        EosTokenId = (uint)metadata["tokenizer.ggml.eos_token_id"];
        var pins = new List<GCHandle>();
        try
        {
            IntPtr[] Pin(List<byte[]> items) => items.Select(b => { var h = GCHandle.Alloc(b, GCHandleType.Pinned); pins.Add(h); return h.AddrOfPinnedObject(); }).ToArray();
            int rc = Native.nfai_tokenizer_create(Pin(tokens), tokens.Select(b => (uint)b.Length).ToArray(), (uint)tokens.Count,
                                                  Pin(merges), merges.Select(b => (uint)b.Length).ToArray(), (uint)merges.Count,
                                                  BosTokenId, EosTokenId, out handle);
            if (rc != 0) throw new InvalidOperationException("nfai_tokenizer_create: malformed vocabulary or merges");
        }
        finally { foreach (var h in pins) h.Free(); }   // the library copies every byte string
    }

    private void Check(int rc)
    {
        if (rc != 0) throw new InvalidOperationException(Marshal.PtrToStringUTF8(Native.nfai_tokenizer_last_error(handle)));
    }

    // Tokenizer.Tokenize(prompt, addBos) (Tokenizer.cs:68-182)
    public List<uint> Tokenize(string prompt, bool addBos = true, bool addEos = false)
    {
        var text = Encoding.UTF8.GetBytes(prompt);
        var ids = new uint[Math.Max(256, 2 * text.Length + 64)];
        Check(Native.nfai_tokenizer_encode_chat(handle, text, (nuint)text.Length, addBos ? 1 : 0, ids, (nuint)ids.Length, out nuint n));
        return ids.Take((int)n).ToList();
    }

    // Tokenizer.Detokenize (Tokenizer.cs:432-462)
    public string Detokenize(IEnumerable<uint> tokenIds)
    {
        var ids = tokenIds.ToArray();
        var buf = new byte[64 + 32 * ids.Length];
        int rc = Native.nfai_tokenizer_decode(handle, ids, (nuint)ids.Length, buf, (nuint)buf.Length, out nuint n);
        if (rc != 0 && (int)n > buf.Length)
        {
            buf = new byte[(int)n];
            rc = Native.nfai_tokenizer_decode(handle, ids, (nuint)ids.Length, buf, (nuint)buf.Length, out n);
        }
        Check(rc);
        return Encoding.UTF8.GetString(buf, 0, (int)n);
    }

    public void Dispose()
    {
        if (handle != IntPtr.Zero) { Native.nfai_tokenizer_destroy(handle); handle = IntPtr.Zero; }
        GC.SuppressFinalize(this);
    }
}
