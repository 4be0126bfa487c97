/*
 * qagg_oracle_impl.h -- the body of the CPU restatement, generic in the element type.  TEST INFRASTRUCTURE ONLY.
 * Included by qagg_oracle.c once per element type with
 *   REAL (float / double), QWORD (uint32_t / uint64_t: QuantizedWordHelper<ElemType>::ValueType, Source/Math/ValueQuantizer.h:39-55),
 *   QSIGNED (its signed twin), QBITS (bits per QWORD), SQRT, and NAME(x) (the symbol x for this element type).
 * The float literals (1e-36f, 0.5f, 2.0f, 4.0f) are the reference's own, in both instantiations.
 */
/* ---- ValueQuantizer<ElemType> (Source/Math/ValueQuantizer.h:58-222) ------------- */
typedef struct
{
    size_t ldNbits;
    size_t Nbits;
    QWORD rangeend;
    REAL quantimin, quantimax, quantimid;
    REAL qfactor, ufactor;
} NAME(valq_t);

/* constructor, ValueQuantizer.h:68-97 */
static void NAME(valq_init)(NAME(valq_t)* q, size_t ldNbits, REAL lower, REAL upper)
{
    q->ldNbits = ldNbits;
    q->Nbits = (size_t) 1 << ldNbits;
    q->quantimin = lower;
    q->quantimax = upper;
    /* a shift by the full word width is forced to 0 (:71-78) */
    q->rangeend = (q->Nbits >= QBITS) ? (QWORD) 0 : ((QWORD) 1 << q->Nbits);
    if (((q->quantimax - q->quantimin) < 1e-36f) || (q->rangeend == 0))
    {
        q->qfactor = q->ufactor = (REAL) 0.0;
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
static QWORD NAME(valq_quantize)(const NAME(valq_t)* q, REAL u, int zeroThr)
{
    if (q->Nbits == QBITS)
    {
        QWORD bits;
        memcpy(&bits, &u, sizeof(bits));
        return bits;
    }
    else if (q->ldNbits == 0)
    {
        int one = zeroThr ? (u >= (REAL) 0.0) : (u >= q->quantimid);
        return one ? (QWORD) 1 : (QWORD) 0;
    }
    else
    {
        if (u <= q->quantimin)
            return 0;
        else if (u >= q->quantimax)
            return q->rangeend - 1;
        else
            return (QWORD) ((QSIGNED) ((u - q->quantimin) * q->qfactor));
    }
}

/* Unquantize, ValueQuantizer.h:131-141 */
static REAL NAME(valq_unquantize)(const NAME(valq_t)* q, QWORD u)
{
    if (q->Nbits == QBITS)
    {
        REAL f;
        memcpy(&f, &u, sizeof(f));
        return f;
    }
    return ((u + (REAL) 0.5) * q->ufactor) + q->quantimin;
}

/* ---- ColumnQuantizer<ElemType> (Source/Math/ColumnQuantizer.h) ------------------- */

/* QWordsPerCol, ColumnQuantizer.h:36-40 */
static size_t NAME(qwords_per_col)(size_t rows, size_t nbits)
{
    const size_t valsPerQWord = QBITS / nbits;
    return (rows + valsPerQWord - 1) / valsPerQWord;
}

/* QuantizedColumnSize, QuantizedMatrix.h:42-47 */
ORACLE_API int64_t NAME(oracle_packed_col_bytes)(int64_t rows, int nbits)
{
    const size_t columnDataSize = ((((size_t) rows * (size_t) nbits) + (QBITS - 1)) / QBITS) * sizeof(QWORD);
    return (int64_t) (2 * sizeof(REAL) + columnDataSize);
}

/* ComputeRangeStatColjSubset with subset 0 of 1 and no-op reducers
 * (ColumnQuantizer.h:80-85, 209-341): sequential fp32 sums, in row order. */
static void NAME(range_stat_col)(const REAL* inMat, const REAL* inResidual, long M, size_t j, size_t bits,
                                 int zeroThr, REAL* lower, REAL* upper)
{
    size_t rows = (size_t) M;
    const REAL* g = inMat + j * rows;
    const REAL* r = inResidual + j * rows;
    REAL mean = 0.0f;
    if (!zeroThr && (bits == 1))
    {
        REAL meanacc = 0.0f;
        for (size_t i = 0; i < rows; i++)
            meanacc += g[i] + r[i];
        mean = meanacc / rows;
    }

    if (bits == 1)
    {
        REAL meanacc0 = 0.0f, meanacc1 = 0.0f;
        unsigned int num0 = 0, num1 = 0;
        for (size_t i = 0; i < rows; i++)
        {
            REAL val = g[i] + r[i];
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
        REAL radius, newmean;
        if (!zeroThr)
        {
            REAL devacc0 = (num0 * mean) - meanacc0;
            REAL devacc1 = meanacc1 - (num1 * mean);
            REAL dev = (devacc0 + devacc1) / rows;
            radius = 2.0f * dev;
            newmean = mean;
        }
        else
        {
            if (num0 == 0)
                num0 = 1;
            if (num1 == 0)
                num1 = 1;
            REAL mean0 = meanacc0 / num0;
            REAL mean1 = meanacc1 / num1;
            newmean = 0.5f * (mean0 + mean1);
            radius = 2.0f * (mean1 - newmean);
        }
        *lower = newmean - radius;
        *upper = newmean + radius;
    }
    else
    {
        REAL stddevs = 4.0f;
        REAL varacc = 0.0f;
        for (size_t i = 0; i < rows; i++)
        {
            REAL val = g[i] + r[i];
            varacc += (val - mean) * (val - mean);
        }
        REAL stddev = SQRT(varacc / rows);
        *lower = mean - (stddevs * stddev);
        *upper = mean + (stddevs * stddev);
    }
}

#ifndef ORACLE_HELPERS_DEFINED
#define ORACLE_HELPERS_DEFINED
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

#endif

/* widths the reference accepts: powers of two up to the word width */
static int NAME(bits_ok)(int nbits)
{
    return nbits >= 1 && nbits <= QBITS && (nbits & (nbits - 1)) == 0;
}

/* MatrixQuantizerCPU::QuantizeAsync (Source/Math/MatrixQuantizerCPU.cpp:12-63) driving
 * ColumnQuantizer::Quantize / QuantizeOneQWord (ColumnQuantizer.h:50-65, 90-147).
 * res_in may alias res_out (the reference's intended use).  Returns 0, or -1 on bad nbits. */
ORACLE_API int NAME(oracle_quantize)(const REAL* grad, const REAL* res_in, REAL* res_out, void* packed,
                                     int64_t M, int64_t N, int nbits, int zeroThr)
{
    if (!NAME(bits_ok)(nbits) || M < 0 || N < 0)
        return -1;
    const size_t ldNbits = ld_of((size_t) nbits);
    const size_t Q = NAME(qwords_per_col)((size_t) M, (size_t) nbits);
    const size_t colBytes = (size_t) NAME(oracle_packed_col_bytes)(M, nbits);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        char* qcol = (char*) packed + j * colBytes;
        REAL lower, upper;
        NAME(range_stat_col)(grad, res_in, (long) M, j, (size_t) nbits, zeroThr, &lower, &upper);
        memcpy(qcol, &lower, sizeof(REAL));
        memcpy(qcol + sizeof(REAL), &upper, sizeof(REAL));
        QWORD* qbits = (QWORD*) (qcol + 2 * sizeof(REAL));

        NAME(valq_t) q;
        NAME(valq_init)(&q, ldNbits, lower, upper);
        for (size_t w = 0; w < Q; w++)
        {
            QWORD bitBuf = 0;
            size_t i = w;
            for (size_t k = 0; (k < QBITS) && (i < (size_t) M); k += (size_t) nbits, i += Q)
            {
                size_t ij = j * (size_t) M + i;
                REAL val = grad[ij] + res_in[ij];
                QWORD qval = NAME(valq_quantize)(&q, val, zeroThr);
                REAL uval = NAME(valq_unquantize)(&q, qval);
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
ORACLE_API int NAME(oracle_unquantize)(const void* packed, REAL* out, int64_t M, int64_t N, int nbits, int add)
{
    if (!NAME(bits_ok)(nbits) || M < 0 || N < 0)
        return -1;
    const size_t ldNbits = ld_of((size_t) nbits);
    const size_t Q = NAME(qwords_per_col)((size_t) M, (size_t) nbits);
    const size_t colBytes = (size_t) NAME(oracle_packed_col_bytes)(M, nbits);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        const char* qcol = (const char*) packed + j * colBytes;
        REAL lower, upper;
        memcpy(&lower, qcol, sizeof(REAL));
        memcpy(&upper, qcol + sizeof(REAL), sizeof(REAL));
        const QWORD* qbits = (const QWORD*) (qcol + 2 * sizeof(REAL));
        NAME(valq_t) q;
        NAME(valq_init)(&q, ldNbits, lower, upper);
        const QWORD bitmask = q.rangeend - 1; /* all ones when rangeend == 0 (full-word pass-through) */
        for (size_t w = 0; w < Q; w++)
        {
            QWORD bitBuf = qbits[w];
            size_t i = w;
            for (size_t k = 0; (k < QBITS) && (i < (size_t) M); k += (size_t) nbits, i += Q)
            {
                const QWORD qval = (bitBuf >> k) & bitmask;
                REAL val = NAME(valq_unquantize)(&q, qval);
                size_t ij = j * (size_t) M + i;
                if (add)
                    val += out[ij];
                out[ij] = val;
            }
        }
    }
    return 0;
}

