/*
 * qagg_oracle.c -- CPU restatement of CNTK's 1-bit-SGD column quantizer.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the shipped library calls it.  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may load it.
 *
 * Parity status: PINNED.  The build recipe next to this file also compiles the
 * reference's own headers (Source/Math/ColumnQuantizer.h, ValueQuantizer.h,
 * QuantizedMatrix.h) in place into oracle/_ref/libqagg_ref.so; the committed
 * fixtures under tests/golden/ were produced by that library and this file must
 * reproduce them byte for byte (tests/test_oracle.py).
 *
 * Every function cites the reference lines it restates (paths relative to the
 * reference project root).  Arithmetic is fp32 with no FMA contraction, the
 * same as the reference CPU build (-msse4.1, Makefile:87): compile with
 * -ffp-contract=off.
 *
 * Layout (Source/Math/QuantizedMatrix.h:27-48): a packed column is
 *   float lower; float upper; uint32 bits[Q];   Q = ceil(M * nbits / 32)
 * and a packed matrix is N such columns back to back (column size 8 + 4Q bytes).
 * Word w of a column holds rows w, w+Q, w+2Q, ... ; the k-th of them at bit
 * k*nbits (Source/Math/ColumnQuantizer.h:50-65, 90-147).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---- ValueQuantizer<float> (Source/Math/ValueQuantizer.h:58-222) ------------- */
typedef struct
{
    size_t ldNbits;
    size_t Nbits;
    uint32_t rangeend;
    float quantimin, quantimax, quantimid;
    float qfactor, ufactor;
} valq_t;

/* constructor, ValueQuantizer.h:68-97 */
static void valq_init(valq_t* q, size_t ldNbits, float lower, float upper)
{
    q->ldNbits = ldNbits;
    q->Nbits = (size_t) 1 << ldNbits;
    q->quantimin = lower;
    q->quantimax = upper;
    /* 1 << 32 is taken mod 32 on the reference's target and then forced to 0 (:71-78) */
    q->rangeend = (q->Nbits >= 32) ? 0u : ((uint32_t) 1 << q->Nbits);
    if (((q->quantimax - q->quantimin) < 1e-36f) || (q->rangeend == 0))
    {
        q->qfactor = q->ufactor = 0.0f;
    }
    else
    {
        size_t usedrangeend = q->rangeend - (q->Nbits > 1);
        q->qfactor = usedrangeend / (q->quantimax - q->quantimin);
        q->ufactor = (q->quantimax - q->quantimin) / usedrangeend;
    }
    q->quantimid = 0.5f * (q->quantimax + q->quantimin);
}

/* Quantize<ZeroThresholdFor1Bit>, ValueQuantizer.h:101-128, 144-156, 195-201 */
static uint32_t valq_quantize(const valq_t* q, float u, int zeroThr)
{
    if (q->Nbits == 32)
    {
        uint32_t bits;
        memcpy(&bits, &u, 4);
        return bits;
    }
    else if (q->ldNbits == 0)
    {
        int one = zeroThr ? (u >= 0.0f) : (u >= q->quantimid);
        return one ? 1u : 0u;
    }
    else
    {
        if (u <= q->quantimin)
            return 0;
        else if (u >= q->quantimax)
            return q->rangeend - 1;
        else
            return (uint32_t) ((int32_t) ((u - q->quantimin) * q->qfactor));
    }
}

/* Unquantize, ValueQuantizer.h:131-141 */
static float valq_unquantize(const valq_t* q, uint32_t u)
{
    if (q->Nbits == 32)
    {
        float f;
        memcpy(&f, &u, 4);
        return f;
    }
    return ((u + 0.5f) * q->ufactor) + q->quantimin;
}

/* ---- ColumnQuantizer<float> (Source/Math/ColumnQuantizer.h) ------------------- */

/* QWordsPerCol, ColumnQuantizer.h:36-40 */
static size_t qwords_per_col(size_t rows, size_t nbits)
{
    const size_t valsPerQWord = 32 / nbits;
    return (rows + valsPerQWord - 1) / valsPerQWord;
}

/* QuantizedColumnSize, QuantizedMatrix.h:42-47 */
ORACLE_API int64_t oracle_packed_col_bytes(int64_t rows, int nbits)
{
    const size_t columnDataSize = ((((size_t) rows * (size_t) nbits) + 31) / 32) * 4;
    return (int64_t) (8 + columnDataSize);
}

/* ComputeRangeStatColjSubset with subset 0 of 1 and no-op reducers
 * (ColumnQuantizer.h:80-85, 209-341): sequential fp32 sums, in row order. */
static void range_stat_col(const float* inMat, const float* inResidual, long M, size_t j, size_t bits,
                           int zeroThr, float* lower, float* upper)
{
    size_t rows = (size_t) M;
    const float* g = inMat + j * rows;
    const float* r = inResidual + j * rows;
    float mean = 0.0f;
    if (!zeroThr && (bits == 1))
    {
        float meanacc = 0.0f;
        for (size_t i = 0; i < rows; i++)
            meanacc += g[i] + r[i];
        mean = meanacc / rows;
    }

    if (bits == 1)
    {
        float meanacc0 = 0.0f, meanacc1 = 0.0f;
        unsigned int num0 = 0, num1 = 0;
        for (size_t i = 0; i < rows; i++)
        {
            float val = g[i] + r[i];
            if (val < mean)
            {
                meanacc0 += val;
                num0++;
            }
            else
            {
                meanacc1 += val;
                num1++;
            }
        }
        float radius, newmean;
        if (!zeroThr)
        {
            float devacc0 = (num0 * mean) - meanacc0;
            float devacc1 = meanacc1 - (num1 * mean);
            float dev = (devacc0 + devacc1) / rows;
            radius = 2.0f * dev;
            newmean = mean;
        }
        else
        {
            if (num0 == 0)
                num0 = 1;
            if (num1 == 0)
                num1 = 1;
            float mean0 = meanacc0 / num0;
            float mean1 = meanacc1 / num1;
            newmean = 0.5f * (mean0 + mean1);
            radius = 2.0f * (mean1 - newmean);
        }
        *lower = newmean - radius;
        *upper = newmean + radius;
    }
    else
    {
        float stddevs = 4.0f;
        float varacc = 0.0f;
        for (size_t i = 0; i < rows; i++)
        {
            float val = g[i] + r[i];
            varacc += (val - mean) * (val - mean);
        }
        float stddev = sqrtf(varacc / rows);
        *lower = mean - (stddevs * stddev);
        *upper = mean + (stddevs * stddev);
    }
}

static size_t ld_of(size_t v)
{
    size_t l = 0;
    while (v > 1)
    {
        v >>= 1;
        l++;
    }
    return l;
}

static int bits_ok(int nbits)
{
    return nbits == 1 || nbits == 2 || nbits == 4 || nbits == 8 || nbits == 16 || nbits == 32;
}

/* MatrixQuantizerCPU::QuantizeAsync (Source/Math/MatrixQuantizerCPU.cpp:12-63) driving
 * ColumnQuantizer::Quantize / QuantizeOneQWord (ColumnQuantizer.h:50-65, 90-147).
 * res_in may alias res_out (the reference's intended use).  Returns 0, or -1 on bad nbits. */
ORACLE_API int oracle_quantize(const float* grad, const float* res_in, float* res_out, void* packed,
                               int64_t M, int64_t N, int nbits, int zeroThr)
{
    if (!bits_ok(nbits) || M < 0 || N < 0)
        return -1;
    const size_t ldNbits = ld_of((size_t) nbits);
    const size_t Q = qwords_per_col((size_t) M, (size_t) nbits);
    const size_t colBytes = (size_t) oracle_packed_col_bytes(M, nbits);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        char* qcol = (char*) packed + j * colBytes;
        float lower, upper;
        range_stat_col(grad, res_in, (long) M, j, (size_t) nbits, zeroThr, &lower, &upper);
        memcpy(qcol, &lower, 4);
        memcpy(qcol + 4, &upper, 4);
        uint32_t* qbits = (uint32_t*) (qcol + 8);

        valq_t q;
        valq_init(&q, ldNbits, lower, upper);
        for (size_t w = 0; w < Q; w++)
        {
            uint32_t bitBuf = 0;
            size_t i = w;
            for (size_t k = 0; (k < 32) && (i < (size_t) M); k += (size_t) nbits, i += Q)
            {
                size_t ij = j * (size_t) M + i;
                float val = grad[ij] + res_in[ij];
                uint32_t qval = valq_quantize(&q, val, zeroThr);
                float uval = valq_unquantize(&q, qval);
                res_out[ij] = val - uval;
                bitBuf |= (qval << k);
            }
            qbits[w] = bitBuf;
        }
    }
    return 0;
}

/* MatrixQuantizerCPU::UnquantizeAsync (MatrixQuantizerCPU.cpp:72-100) driving
 * ColumnQuantizer::Unquantize / UnquantizeOneQWord (ColumnQuantizer.h:69-77, 150-203). */
ORACLE_API int oracle_unquantize(const void* packed, float* out, int64_t M, int64_t N, int nbits, int add)
{
    if (!bits_ok(nbits) || M < 0 || N < 0)
        return -1;
    const size_t ldNbits = ld_of((size_t) nbits);
    const size_t Q = qwords_per_col((size_t) M, (size_t) nbits);
    const size_t colBytes = (size_t) oracle_packed_col_bytes(M, nbits);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        const char* qcol = (const char*) packed + j * colBytes;
        float lower, upper;
        memcpy(&lower, qcol, 4);
        memcpy(&upper, qcol + 4, 4);
        const uint32_t* qbits = (const uint32_t*) (qcol + 8);
        valq_t q;
        valq_init(&q, ldNbits, lower, upper);
        const uint32_t bitmask = q.rangeend - 1; /* all ones when rangeend == 0 (32-bit pass-through) */
        for (size_t w = 0; w < Q; w++)
        {
            uint32_t bitBuf = qbits[w];
            size_t i = w;
            for (size_t k = 0; (k < 32) && (i < (size_t) M); k += (size_t) nbits, i += Q)
            {
                const uint32_t qval = (bitBuf >> k) & bitmask;
                float val = valq_unquantize(&q, qval);
                size_t ij = j * (size_t) M + i;
                if (add)
                    val += out[ij];
                out[ij] = val;
            }
        }
    }
    return 0;
}

/* GetStripeForNode (Source/1BitSGD/AllReduceDistGradAggregator.h:56-65,
 * Source/1BitSGD/QuantizedDistributedCommunicator.h:158-165). */
ORACLE_API void oracle_stripe(int64_t numCols, int64_t nodeRank, int64_t numNodes, int64_t* start, int64_t* n)
{
    int64_t per = numCols / numNodes;
    int64_t residue = numCols % numNodes;
    *start = per * nodeRank + (residue < nodeRank ? residue : nodeRank);
    *n = per + ((nodeRank < residue) ? 1 : 0);
}
