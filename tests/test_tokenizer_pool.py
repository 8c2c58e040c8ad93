import asyncio

from axon_b200.utils.tokenizer import ByteTokenizer
from axon_b200.utils.tokenizer_pool import TokenizerPool


def test_tokenizer_pool_async_and_sync():
    tok = ByteTokenizer()
    pool = TokenizerPool(tok, tokenizer_path="byte-tokenizer", num_workers=2)
    texts = [f"hello <|im_end|> number {i} é" for i in range(7)]

    async def go():
        await pool.start()
        ids = await pool.encode(texts[0])
        assert ids == tok.encode(texts[0]) and await pool.decode(ids) == texts[0]
        b = await pool.batch_encode(texts)
        assert b == [tok.encode(t) for t in texts]
        assert await pool.batch_decode(b) == texts
        i2, strs = await pool.encode_with_strs(texts[1])
        assert i2 == b[1] and len(strs) == len(i2)
        many = await asyncio.gather(*(pool.encode(t) for t in texts * 5))
        assert many == b * 5
    try:
        asyncio.run(go())
        assert pool.encode_sync("abc") == tok.encode("abc") and pool.decode_sync([104, 105]) == "hi"
        assert pool.batch_encode_sync(texts) == [tok.encode(t) for t in texts]
        assert pool.eos_token_id == tok.eos_token_id and pool.num_workers == 2 and pool.batch_decode_sync([]) == []
    finally:
        pool.shutdown_sync()
