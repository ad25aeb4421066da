/* Embeds the sm_100a cubin built from kernels/optim_kernels.cu into the library.
 * OE_CUBIN_PATH is given on the command line by the Makefile. */
    .section .rodata
    .balign 64
    .global oe_cubin_start
    .global oe_cubin_end
oe_cubin_start:
    .incbin OE_CUBIN_PATH
oe_cubin_end:
    .byte 0
    .section .note.GNU-stack,"",@progbits
