/* A plain C99 client of the library: what a cgo / Rust-FFI / C caller sees. Includes the header as C,
 * links against liblbk.so and calls the entry points that need no GPU: the ABI version, the layout
 * helpers of pack.rs:18-24,83-85, and the error convention (status code + lbk_last_error, no abort) on
 * null arguments. Built and run by tests/test_abi_symbols.py. */
#include <stdio.h>
#include <string.h>

#include "lbk.h"

int main(void) {
    int bad = 0;
    if (lbk_abi_version() != 1) { printf("abi version %d\n", lbk_abi_version()); bad++; }
    if (lbk_padded_cols(2560) != 2560 || lbk_padded_cols(129) != 256 || lbk_padded_cols(0) != 0) { printf("padded_cols\n"); bad++; }
    if (lbk_row_bytes(2560) != 640 || lbk_row_bytes(6912) != 1728 || lbk_row_bytes(1) != 32) { printf("row_bytes\n"); bad++; }
    /* a null context is a status code and a message, never a crash */
    {
        lbk_weight *w = NULL;
        unsigned char bytes[32];
        int st;
        memset(bytes, 0x55, sizeof bytes);
        st = lbk_weight_upload(NULL, 1, 128, bytes, sizeof bytes, 1.0f, &w);
        if (st == LBK_OK || w != NULL) { printf("null context accepted\n"); bad++; }
        if (lbk_last_error() == NULL || strlen(lbk_last_error()) == 0) { printf("no message\n"); bad++; }
    }
    printf(bad ? "FAILED\n" : "C client ok\n");
    return bad;
}
